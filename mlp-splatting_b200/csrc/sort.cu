// Per-tile depth sort: key = t* of the tile-centre ray against each candidate
// (scannet/cuda/np_tile_kernels.cu:483-518), stable ascending order (1914-1990).
// Keys are positive floats (or the 1e30 sentinel), so their bit patterns order like the values and the
// sort runs on the raw bits: a bitonic network in shared memory over the 64-bit composite (key bits,
// tie-break); lists of up to 512 candidates are sorted by one warp (eight tiles per CTA), longer
// lists by a whole CTA.
#include "frame.cuh"

namespace mlpsp {

constexpr int kSortCap = 2048;

// ---- warp-level bitonic sort in shared memory: N (a power of two >= 32) elements per warp ----
// Compare-exchange t of a stage works on elements i and i | j, where i is t with a zero bit inserted
// at the position of j.  One __syncwarp per stage, no block barrier: eight tiles sort side by side
// in one 256-thread CTA.
template <typename T, int N, int THREADS = 32>
__device__ __forceinline__ void warp_bitonic(T* buf) {
  const int lane = threadIdx.x & (THREADS - 1);
  constexpr int PER = (N / 2 + THREADS - 1) / THREADS;   // compare-exchanges per thread and stage
#pragma unroll 1
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll 1
    for (int j = k >> 1; j > 0; j >>= 1) {
      T a[PER], b[PER];
      int ia[PER];
      // all loads of the stage first, so their shared-memory latencies overlap
#pragma unroll
      for (int q = 0; q < PER; ++q) {
        const int t = q * THREADS + lane;
        ia[q] = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        if (N >= 2 * THREADS || t < N / 2) { a[q] = buf[ia[q]]; b[q] = buf[ia[q] | j]; }
      }
#pragma unroll
      for (int q = 0; q < PER; ++q) {
        const int t = q * THREADS + lane;
        if (N >= 2 * THREADS || t < N / 2) {
          const bool up = (ia[q] & k) == 0;
          if (up ? (a[q] > b[q]) : (a[q] < b[q])) { buf[ia[q]] = b[q]; buf[ia[q] | j] = a[q]; }
        }
      }
      if (THREADS == 32) __syncwarp(); else __syncthreads();
    }
  }
}

// One warp sorts one tile of at most N candidates in its own slice of shared memory by the
// composite (depth key bits, tie-break).  FROM_SCATTER: the list comes straight from the binning
// scatter in arbitrary order and holds distinct ids, so the id itself is the tie-break: the result is
// the stable sort of the ascending-id list, and the id is read back from the sorted composite.
// Otherwise the tie-break is the position in the caller's list (stable sort of that list).
template <int N, bool FROM_SCATTER>
__device__ __forceinline__ void warp_sort_tile(unsigned long long* buf, const float4* __restrict__ geom, int n,
                                               const int32_t* tile_prims, int32_t* __restrict__ sorted_prims,
                                               float* __restrict__ keys_out, int s, int len, V3 o, V3 d, int key_mode) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i0 = 0; i0 < N; i0 += 32) {
    const int i = i0 + lane;
    unsigned long long kv = ~0ull;
    if (i < len) {
      const int p = tile_prims[s + i];
      float key = MLPSP_SENTINEL_KEY;
      if (p >= 0 && p < n) {
        const Geom g = load_geom(geom, p);
        key = key_mode ? tile_key_euclid(g, o, d) : tile_key(g, o, d);
      }
      kv = ((unsigned long long)__float_as_uint(key) << 32) | (unsigned long long)(uint32_t)(FROM_SCATTER ? p : i);
    }
    buf[i] = kv;
  }
  __syncwarp();
  warp_bitonic<unsigned long long, N>(buf);
  for (int i = lane; i < len; i += 32) {
    const unsigned long long kv = buf[i];
    sorted_prims[s + i] = FROM_SCATTER ? (int32_t)(uint32_t)kv : tile_prims[s + (int)(uint32_t)kv];
    if (keys_out) keys_out[s + i] = __uint_as_float((uint32_t)(kv >> 32));
  }
}

// Block-wide path for long lists: the same bitonic network run by 256 threads on N = 1024 or 2048 slots.
template <int THREADS, int N, bool FROM_SCATTER>
__device__ __forceinline__ void block_sort_tile(unsigned long long* buf, const float4* __restrict__ geom, int n,
                                                const int32_t* tile_prims, int32_t* __restrict__ sorted_prims,
                                                float* __restrict__ keys_out, int s, int len, V3 o, V3 d, int key_mode) {
  for (int i = threadIdx.x; i < N; i += THREADS) {
    unsigned long long kv = ~0ull;
    if (i < len) {
      const int p = tile_prims[s + i];
      float key = MLPSP_SENTINEL_KEY;
      if (p >= 0 && p < n) {
        const Geom g = load_geom(geom, p);
        key = key_mode ? tile_key_euclid(g, o, d) : tile_key(g, o, d);
      }
      kv = ((unsigned long long)__float_as_uint(key) << 32) | (unsigned long long)(uint32_t)(FROM_SCATTER ? p : i);
    }
    buf[i] = kv;
  }
  __syncthreads();
  warp_bitonic<unsigned long long, N, THREADS>(buf);
  for (int i = threadIdx.x; i < len; i += THREADS) {
    const unsigned long long kv = buf[i];
    sorted_prims[s + i] = FROM_SCATTER ? (int32_t)(uint32_t)kv : tile_prims[s + (int)(uint32_t)kv];
    if (keys_out) keys_out[s + i] = __uint_as_float((uint32_t)(kv >> 32));
  }
  __syncthreads();
}

constexpr int kTilesPerCta = 8;
constexpr int kWarpSortMax = 512;

// Short lists: one warp per tile, eight tiles per CTA.  Tiles with more than kWarpSortMax candidates
// are appended to long_list for k_sort_long, so that each of them gets a CTA of its own (they hold
// most of the candidates and sit next to each other in the image).
template <bool IDSORT>
__global__ void __launch_bounds__(256) k_sort_tiles(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, const int32_t* tile_prims, int W, int H, int ts, int ntx, int T, int cap,
    int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out, int key_mode, int32_t* __restrict__ long_list,
    int32_t* __restrict__ long_count, const int32_t* __restrict__ status) {
  __shared__ __align__(16) unsigned long long s_buf[kTilesPerCta * kWarpSortMax];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * kTilesPerCta + warp;
  if (tile >= T) return;
  const int s = tile_offsets[tile];
  const int len = min(tile_offsets[tile + 1] - s, cap);
  if (len <= 0) return;
  if (len > kWarpSortMax) {
    if (lane == 0) long_list[atomicAdd(long_count, 1)] = tile;
    return;
  }
  const int tx = tile % ntx, ty = tile / ntx;
  const int cx = min(tx * ts + (ts >> 1), W - 1), cy = min(ty * ts + (ts >> 1), H - 1);
  const int64_t pc = (int64_t)cy * W + cx;
  const V3 o = load3(rays_o, pc), d = load3(rays_d, pc);
  unsigned long long* buf = s_buf + warp * kWarpSortMax;
  if (len <= 64) warp_sort_tile<64, IDSORT>(buf, geom, n, tile_prims, sorted_prims, keys_out, s, len, o, d, key_mode);
  else if (len <= 128) warp_sort_tile<128, IDSORT>(buf, geom, n, tile_prims, sorted_prims, keys_out, s, len, o, d, key_mode);
  else if (len <= 256) warp_sort_tile<256, IDSORT>(buf, geom, n, tile_prims, sorted_prims, keys_out, s, len, o, d, key_mode);
  else warp_sort_tile<512, IDSORT>(buf, geom, n, tile_prims, sorted_prims, keys_out, s, len, o, d, key_mode);
}

// Long lists: one CTA per tile of long_list (grid-stride), block-wide radix sort.
template <int THREADS, int CAP, bool IDSORT>
__global__ void __launch_bounds__(THREADS) k_sort_long(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, const int32_t* tile_prims, int W, int H, int ts, int ntx,
    int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out, int key_mode,
    const int32_t* __restrict__ long_list, const int32_t* __restrict__ long_count,
    const int32_t* __restrict__ status) {
  __shared__ __align__(16) unsigned long long s_buf[CAP];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int count = *long_count;
  for (int q = blockIdx.x; q < count; q += gridDim.x) {
    const int tile = long_list[q];
    const int s = tile_offsets[tile];
    const int len = min(tile_offsets[tile + 1] - s, CAP);
    const int tx = tile % ntx, ty = tile / ntx;
    const int cx = min(tx * ts + (ts >> 1), W - 1), cy = min(ty * ts + (ts >> 1), H - 1);
    const int64_t pc = (int64_t)cy * W + cx;
    const V3 o = load3(rays_o, pc), d = load3(rays_d, pc);
    if (len <= CAP / 2)
      block_sort_tile<THREADS, CAP / 2, IDSORT>(s_buf, geom, n, tile_prims, sorted_prims, keys_out, s, len, o, d, key_mode);
    else
      block_sort_tile<THREADS, CAP, IDSORT>(s_buf, geom, n, tile_prims, sorted_prims, keys_out, s, len, o, d, key_mode);
  }
}

int launch_sort(const mlpsp_scene* sc, const mlpsp_frame* fr, float* keys_out, cudaStream_t st, bool unordered_input,
                int32_t* long_list, int32_t* long_count) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  const int ntx = (fr->width + fr->tile - 1) / fr->tile;
  MLPSP_REQUIRE(fr->tile_capacity > 0 && fr->tile_capacity <= kSortCap, MLPSP_E_LIMIT,
                "tile_capacity must be in [1, %d]", kSortCap);
  MLPSP_REQUIRE(long_list && long_count, MLPSP_E_ARG, "sort: scratch for the long-tile list missing");
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  MLPSP_CUDA_OK(cudaMemsetAsync(long_count, 0, 4, st));
  LaunchScope scope(kKSort, 2, st);
  const int grid = (T + kTilesPerCta - 1) / kTilesPerCta;
  const int grid_long = std::min(T, sms * 6);
  const float4* geom = (const float4*)sc->geom;
  if (unordered_input) {
    k_sort_tiles<true><<<grid, 256, 0, st>>>(fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets, fr->tile_prims,
                                             fr->width, fr->height, fr->tile, ntx, T, kSortCap, fr->sorted_prims, keys_out,
                                             fr->sort_key, long_list, long_count, fr->status);
    k_sort_long<256, kSortCap, true><<<grid_long, 256, 0, st>>>(fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets,
                                                               fr->tile_prims, fr->width, fr->height, fr->tile, ntx,
                                                               fr->sorted_prims, keys_out, fr->sort_key, long_list,
                                                               long_count, fr->status);
  } else {
    k_sort_tiles<false><<<grid, 256, 0, st>>>(fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets, fr->tile_prims,
                                              fr->width, fr->height, fr->tile, ntx, T, kSortCap, fr->sorted_prims, keys_out,
                                              fr->sort_key, long_list, long_count, fr->status);
    k_sort_long<256, kSortCap, false><<<grid_long, 256, 0, st>>>(fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets,
                                                                fr->tile_prims, fr->width, fr->height, fr->tile, ntx,
                                                                fr->sorted_prims, keys_out, fr->sort_key, long_list,
                                                                long_count, fr->status);
  }
  return cuda_check(cudaGetLastError(), "sort_tiles");
}

}  // namespace mlpsp
