// Per-tile depth sort: key = t* of the tile-centre ray against each candidate
// (scannet/cuda/np_tile_kernels.cu:483-518), stable ascending order (1914-1990).
// Keys are positive floats (or the 1e30 sentinel), so their bit patterns order like the values and
// the block radix sort runs on the raw bits.
#include "frame.cuh"
#include "block_sort.cuh"

namespace mlpsp {

constexpr int kSortCap = 2048;

// IDSORT: the incoming list is in arbitrary order (straight from the binning scatter); it is first put
// in ascending id order (written back as the canonical tile list), then sorted by key, in one kernel.
template <int THREADS, int CAP, bool IDSORT>
__global__ void __launch_bounds__(THREADS) k_sort_tiles(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, int32_t* __restrict__ tile_prims, int W, int H, int ts, int ntx,
    int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out, int key_mode,
    const int32_t* __restrict__ status) {
  using Sort = BlockRadixSort<THREADS, CAP>;
  __shared__ typename Sort::Smem sm;
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tile = blockIdx.x;
  const int s = tile_offsets[tile], e = tile_offsets[tile + 1];
  const int len = min(e - s, CAP);
  if (len <= 0) return;
  const int tx = tile % ntx, ty = tile / ntx;
  const int cx = min(tx * ts + (ts >> 1), W - 1), cy = min(ty * ts + (ts >> 1), H - 1);
  const int64_t pc = (int64_t)cy * W + cx;
  const V3 o = load3(rays_o, pc), d = load3(rays_d, pc);
  int src = 0;
  if (IDSORT) {
    for (int i = threadIdx.x; i < len; i += THREADS) {
      const int32_t p = tile_prims[s + i];
      sm.key[0][i] = (uint32_t)p;
      sm.val[0][i] = p;
    }
    __syncthreads();
    src = Sort::sort(sm, len);
    for (int i = threadIdx.x; i < len; i += THREADS) tile_prims[s + i] = sm.val[src][i];
  }
  for (int i = threadIdx.x; i < len; i += THREADS) {
    const int p = IDSORT ? sm.val[src][i] : tile_prims[s + i];
    float key = MLPSP_SENTINEL_KEY;
    if (p >= 0 && p < n) {
      const Geom g = load_geom(geom, p);
      key = key_mode ? tile_key_euclid(g, o, d) : tile_key(g, o, d);
    }
    sm.key[0][i] = __float_as_uint(key);
    sm.val[0][i] = p;
  }
  __syncthreads();
  const int cur = Sort::sort(sm, len);
  for (int i = threadIdx.x; i < len; i += THREADS) {
    sorted_prims[s + i] = sm.val[cur][i];
    if (keys_out) keys_out[s + i] = __uint_as_float(sm.key[cur][i]);
  }
}

int launch_sort(const mlpsp_scene* sc, const mlpsp_frame* fr, float* keys_out, cudaStream_t st, bool unordered_input) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  const int ntx = (fr->width + fr->tile - 1) / fr->tile;
  MLPSP_REQUIRE(fr->tile_capacity > 0 && fr->tile_capacity <= kSortCap, MLPSP_E_LIMIT,
                "tile_capacity must be in [1, %d]", kSortCap);
  LaunchScope scope(kKSort, 1, st);
  if (unordered_input)
    k_sort_tiles<256, kSortCap, true><<<T, 256, 0, st>>>(fr->rays_o, fr->rays_d, (const float4*)sc->geom, sc->n,
                                                        fr->tile_offsets, fr->tile_prims, fr->width, fr->height,
                                                        fr->tile, ntx, fr->sorted_prims, keys_out, fr->sort_key,
                                                        fr->status);
  else
    k_sort_tiles<256, kSortCap, false><<<T, 256, 0, st>>>(fr->rays_o, fr->rays_d, (const float4*)sc->geom, sc->n,
                                                         fr->tile_offsets, fr->tile_prims, fr->width, fr->height,
                                                         fr->tile, ntx, fr->sorted_prims, keys_out, fr->sort_key,
                                                         fr->status);
  return cuda_check(cudaGetLastError(), "sort_tiles");
}

}  // namespace mlpsp
