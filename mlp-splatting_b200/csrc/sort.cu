// Per-tile depth sort: key = t* of the tile-centre ray against each candidate
// (scannet/cuda/np_tile_kernels.cu:483-518), stable ascending order (1914-1990).
// Keys are positive floats (or the 1e30 sentinel), so their bit patterns order like the values and the
// sort runs on the raw bits: a bitonic network over the 64-bit composite (key bits, tie-break); lists of up
// to 256 candidates are sorted by one warp in registers (eight tiles per CTA), longer lists by a whole CTA in
// shared memory.
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

// Composite of one candidate: (depth key bits << 32) | tie-break.  FROM_SCATTER: the list comes straight
// from the binning scatter in arbitrary order and holds distinct ids, so the id itself is the tie-break
// (the result is the stable sort of the ascending-id list) and the id is read back from the sorted
// composite.  Otherwise the tie-break is the position in the caller's list (stable sort of that list).
template <bool FROM_SCATTER>
__device__ __forceinline__ unsigned long long make_composite(const float4* __restrict__ geom, int n, int p, int i, V3 o,
                                                             V3 d, int key_mode) {
  float key = MLPSP_SENTINEL_KEY;
  if (p >= 0 && p < n) {
    // key_mode 2 (per-pixel ordering): the pixels sort their own hits later and fall back on the list order for
    // equal hit distances (rays that start inside several primitives meet them all at t = 0), so the list keeps
    // the order it was given, or ascending ids when it comes from the binning scatter.  Bit 2 (value 4) asks for the
    // tile-centre key in the reference kernels' arithmetic (frame.hit_arith = 1).
    if (key_mode == 4) {
      key = tile_key_ref(load_geom_ref(geom, p), o, d);
    } else {
      const Geom g = load_geom(geom, p);
      key = (key_mode & 3) == 2 ? 0.f : ((key_mode & 3) ? tile_key_euclid(g, o, d) : tile_key(g, o, d));
    }
  }
  return ((unsigned long long)__float_as_uint(key) << 32) | (unsigned long long)(uint32_t)(FROM_SCATTER ? p : i);
}

// sorted_prims[s .. s + len) = the sorted list; [s + len, s + span) = -1 (span > len only after a
// pre-tested binning, whose dropped pairs leave the end of the tile's span unused)
template <bool FROM_SCATTER>
__device__ __forceinline__ void write_sorted(const unsigned long long* buf, const int32_t* tile_prims,
                                             int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out, int s,
                                             int len, int span, int first, int step) {
  for (int i = first; i < span; i += step) {
    if (i < len) {
      const unsigned long long kv = buf[i];
      sorted_prims[s + i] = FROM_SCATTER ? (int32_t)(uint32_t)kv : tile_prims[s + (int)(uint32_t)kv];
      if (keys_out) keys_out[s + i] = __uint_as_float((uint32_t)(kv >> 32));
    } else {
      sorted_prims[s + i] = -1;
    }
  }
}

constexpr int kTilesPerCta = 8;
constexpr int kWarpSortMax = 256;

// ---- warp-level bitonic sort in registers: lane l holds the elements r * 32 + l, r < PER ----
// A compare-exchange at distance j >= 32 pairs two registers of the same lane; at distance j < 32 it pairs the same
// register of the lanes l and l ^ j, one shuffle each way.  Ascending where the element index has bit k clear.
// No shared memory and no barrier: the stages of a tile follow one another at the latency of a shuffle.
__device__ __forceinline__ unsigned long long shfl_xor_u64(unsigned long long v, int j) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, (uint32_t)v, j);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, (uint32_t)(v >> 32), j);
  return ((unsigned long long)hi << 32) | lo;
}

template <int PER>
__device__ __forceinline__ void warp_bitonic_regs(unsigned long long (&v)[PER], int lane) {
  constexpr int N = PER * 32;
#pragma unroll
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 32) {
        const int jr = j >> 5;
#pragma unroll
        for (int r = 0; r < PER; ++r) {
          if ((r & jr) == 0) {
            const bool up = ((r * 32) & k) == 0;          // k >= 64 here: the lane bits do not reach it
            const unsigned long long a = v[r], b = v[r | jr];
            const bool swap = up ? (a > b) : (a < b);
            v[r] = swap ? b : a;
            v[r | jr] = swap ? a : b;
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
          const unsigned long long a = v[r];
          const unsigned long long b = shfl_xor_u64(a, j);
          const bool up = ((r * 32 + lane) & k) == 0;
          const bool lower = (lane & j) == 0;
          const bool keep_min = lower == up;
          const unsigned long long mn = a < b ? a : b, mx = a < b ? b : a;
          v[r] = keep_min ? mn : mx;
        }
      }
    }
  }
}

// ---- CTA-level bitonic sort, PER elements per thread in registers: thread t holds the elements t * PER + r ----
// Distances below PER stay inside a thread, distances below 32 * PER pair two lanes of a warp (shuffles); only the
// remaining distances (6 of the 45 stages of a 512-element sort, 10 of 55 at 1,024) cross warps and go through
// shared memory between two CTA barriers.  buf holds the elements on entry and, sorted, on return.
template <int PER, int THREADS>
__device__ __forceinline__ void cta_bitonic_hybrid(unsigned long long* buf) {
  constexpr int N = PER * THREADS;
  const int tid = threadIdx.x;
  unsigned long long v[PER];
#pragma unroll
  for (int r = 0; r < PER; ++r) v[r] = buf[tid * PER + r];
  __syncthreads();
#pragma unroll
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j < PER) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
          if ((r & j) == 0) {
            const bool up = ((tid * PER + r) & k) == 0;
            const unsigned long long a = v[r], b = v[r | j];
            const bool swap = up ? (a > b) : (a < b);
            v[r] = swap ? b : a;
            v[r | j] = swap ? a : b;
          }
        }
      } else if (j < 32 * PER) {
        const int jl = j / PER;
#pragma unroll
        for (int r = 0; r < PER; ++r) {
          const unsigned long long a = v[r];
          const unsigned long long b = shfl_xor_u64(a, jl);
          const bool up = ((tid * PER + r) & k) == 0;
          const bool keep_min = ((tid & jl) == 0) == up;
          const unsigned long long mn = a < b ? a : b, mx = a < b ? b : a;
          v[r] = keep_min ? mn : mx;
        }
      } else {
#pragma unroll
        for (int r = 0; r < PER; ++r) buf[tid * PER + r] = v[r];
        __syncthreads();
#pragma unroll
        for (int r = 0; r < PER; ++r) {
          const int e = tid * PER + r;
          const unsigned long long a = v[r], b = buf[e ^ j];
          const bool keep_min = ((e & j) == 0) == ((e & k) == 0);
          const unsigned long long mn = a < b ? a : b, mx = a < b ? b : a;
          v[r] = keep_min ? mn : mx;
        }
        __syncthreads();
      }
    }
  }
#pragma unroll
  for (int r = 0; r < PER; ++r) buf[tid * PER + r] = v[r];
  __syncthreads();
}

// One tile's list (len <= PER * 32) sorted by one warp in registers and written out.
template <int PER, bool FROM_SCATTER>
__device__ __forceinline__ void sort_tile_in_registers(const float4* __restrict__ geom, int n, const int32_t* tile_prims,
                                                       int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out,
                                                       int s, int len, int span, V3 o, V3 d, int key_mode, int lane) {
  unsigned long long v[PER];
#pragma unroll
  for (int r = 0; r < PER; ++r) {
    const int e = r * 32 + lane;
    v[r] = e < len ? make_composite<FROM_SCATTER>(geom, n, tile_prims[s + e], e, o, d, key_mode) : ~0ull;
  }
  warp_bitonic_regs<PER>(v, lane);
#pragma unroll
  for (int r = 0; r < PER; ++r) {
    const int e = r * 32 + lane;
    if (e < len) {
      sorted_prims[s + e] = FROM_SCATTER ? (int32_t)(uint32_t)v[r] : tile_prims[s + (int)(uint32_t)v[r]];
      if (keys_out) keys_out[s + e] = __uint_as_float((uint32_t)(v[r] >> 32));
    }
  }
  for (int i = len + lane; i < span; i += 32) sorted_prims[s + i] = -1;
}

// end of k_sort_tiles: the grid may not complete before the grid it was launched behind has
__device__ __forceinline__ void sort_tiles_done() {
  if ((threadIdx.x & 31) == 0) chain_wait();
}

// Short lists: one warp per tile, eight tiles per CTA.  Tiles with more than kWarpSortMax candidates are left to
// k_sort_long, which gives each of them a CTA of its own.
template <bool IDSORT>
__global__ void __launch_bounds__(256, 6) k_sort_tiles(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, const int32_t* tile_prims, int W, int H, int ts, int ntx, int T, int cap,
    int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out, int key_mode, int32_t* __restrict__ long_list,
    int32_t* __restrict__ long_count, const int32_t* __restrict__ list_len, int32_t* __restrict__ status) {
  // Launched behind k_sort_long as its programmatic dependent WITHOUT waiting for it here: the two kernels sort
  // disjoint tiles and run side by side.  What this kernel reads (the binned lists, the status word) was complete
  // before k_sort_long's CTAs got past their own wait, and none of this kernel's CTAs starts before all of them
  // have.  The wait is at the end instead (sort_tiles_done), so that this grid's completion implies the other's.
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) { sort_tiles_done(); return; }
  const int lane = threadIdx.x & 31;
  // warps draw tiles from a shared cursor (long_count[1]): list lengths differ by two orders of magnitude, and
  // a fixed deal would leave most warps of a CTA waiting for the one with the longest list
  for (;;) {
  int tile = 0;
  if (lane == 0) tile = atomicAdd(long_count + 1, 1);
  tile = __shfl_sync(0xffffffffu, tile, 0);
  if (tile >= T) { sort_tiles_done(); return; }
  const int s = tile_offsets[tile];
  const int span = min(tile_offsets[tile + 1] - s, cap);
  const int len = list_len ? min(list_len[tile], span) : span;
  if (list_len && lane == 0 && len > 0) atomicAdd(status + MLPSP_ST_PAIRS_KEPT, len);
  if (len > kWarpSortMax) continue;      // k_sort_long's
  if (len <= 0) {
    for (int i = lane; i < span; i += 32) sorted_prims[s + i] = -1;
    continue;
  }
  const int tx = tile % ntx, ty = tile / ntx;
  const int cx = min(tx * ts + (ts >> 1), W - 1), cy = min(ty * ts + (ts >> 1), H - 1);
  const int64_t pc = (int64_t)cy * W + cx;
  const V3 o = load3(rays_o, pc), d = load3(rays_d, pc);
  if (len <= 32) sort_tile_in_registers<1, IDSORT>(geom, n, tile_prims, sorted_prims, keys_out, s, len, span, o, d, key_mode, lane);
  else if (len <= 64) sort_tile_in_registers<2, IDSORT>(geom, n, tile_prims, sorted_prims, keys_out, s, len, span, o, d, key_mode, lane);
  else if (len <= 128) sort_tile_in_registers<4, IDSORT>(geom, n, tile_prims, sorted_prims, keys_out, s, len, span, o, d, key_mode, lane);
  else sort_tile_in_registers<8, IDSORT>(geom, n, tile_prims, sorted_prims, keys_out, s, len, span, o, d, key_mode, lane);
  }
}

// Long lists (more than kWarpSortMax candidates): one CTA per such tile, the same bitonic network with the elements in
// the registers of the CTA's threads (cta_bitonic_hybrid).  Launched before k_sort_tiles, which runs beside it.
template <int THREADS, int CAP, bool IDSORT>
__global__ void __launch_bounds__(THREADS) k_sort_long(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, const int32_t* tile_prims, int W, int H, int ts, int ntx,
    int32_t* __restrict__ sorted_prims, float* __restrict__ keys_out, int key_mode, int T,
    int32_t* __restrict__ cursor, const int32_t* __restrict__ list_len, const int32_t* __restrict__ status) {
  __shared__ __align__(16) unsigned long long s_buf[CAP];
  __shared__ int s_tile;
  chain_wait();
  chain_release();
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  // CTAs draw tiles one at a time from a shared cursor: long lists cluster in the dense part of the image (on the
  // 100,000-primitive bench frame 2,301 of 12,750 tiles hold more than 256 candidates), so a fixed deal leaves
  // most CTAs idle behind the ones that met several
  for (;;) {
    if (threadIdx.x == 0) s_tile = atomicAdd(cursor, 1);
    __syncthreads();
    const int tile = s_tile;
    __syncthreads();
    if (tile >= T) return;
    const int s = tile_offsets[tile];
    const int span = min(tile_offsets[tile + 1] - s, CAP);
    const int len = list_len ? min(list_len[tile], span) : span;
    if (len <= kWarpSortMax) continue;        // k_sort_tiles' (uniform over the CTA)
    const int tx = tile % ntx, ty = tile / ntx;
    const int cx = min(tx * ts + (ts >> 1), W - 1), cy = min(ty * ts + (ts >> 1), H - 1);
    const int64_t pc = (int64_t)cy * W + cx;
    const V3 o = load3(rays_o, pc), d = load3(rays_d, pc);
    const int N = len <= CAP / 4 ? CAP / 4 : (len <= CAP / 2 ? CAP / 2 : CAP);
    for (int i = threadIdx.x; i < N; i += THREADS)
      s_buf[i] = (i < len) ? make_composite<IDSORT>(geom, n, tile_prims[s + i], i, o, d, key_mode) : ~0ull;
    __syncthreads();
    if (N == CAP / 4) cta_bitonic_hybrid<CAP / 4 / THREADS, THREADS>(s_buf);
    else if (N == CAP / 2) cta_bitonic_hybrid<CAP / 2 / THREADS, THREADS>(s_buf);
    else warp_bitonic<unsigned long long, CAP, THREADS>(s_buf);      // beyond 1,024 candidates: rare, in shared memory
    write_sorted<IDSORT>(s_buf, tile_prims, sorted_prims, keys_out, s, len, span, threadIdx.x, THREADS);
    __syncthreads();
  }
}

// ---- per-tile ray frames for the tile pre-test: one warp per tile, two pixels per lane ----
__global__ void __launch_bounds__(256) k_tile_frames(const float* __restrict__ rays_o, const float* __restrict__ rays_d,
                                                     int W, int H, int ntx, int T, TileFrame* __restrict__ frames) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * 8 + warp;
  if (tile >= T) return;
  const int tx = tile % ntx, ty = tile / ntx;
  V3 dd[2];
  bool same = true;
  const int64_t p0 = (int64_t)min(ty * 8, H - 1) * W + min(tx * 8, W - 1);
  const V3 o0 = load3(rays_o, p0);
  float sx = 0.f, sy = 0.f, sz = 0.f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int k = h * 32 + lane;
    // pixels past the image edge repeat the edge pixel: they add no new ray
    const int64_t pix = (int64_t)min(ty * 8 + (k >> 3), H - 1) * W + min(tx * 8 + (k & 7), W - 1);
    const V3 o = load3(rays_o, pix);
    dd[h] = load3(rays_d, pix);
    same = same && o.x == o0.x && o.y == o0.y && o.z == o0.z;
    sx += dd[h].x; sy += dd[h].y; sz += dd[h].z;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    sx += __shfl_xor_sync(0xffffffffu, sx, off);
    sy += __shfl_xor_sync(0xffffffffu, sy, off);
    sz += __shfl_xor_sync(0xffffffffu, sz, off);
  }
  const float inv = rsqrtf(sx * sx + sy * sy + sz * sz);
  const float ax = sx * inv, ay = sy * inv, az = sz * inv;
  // u: the image's x direction made orthogonal to a (direction of pixel 7 minus pixel 0 of the first row);
  // a fixed axis when the tile is one pixel wide
  const int64_t p7 = (int64_t)min(ty * 8, H - 1) * W + min(tx * 8 + 7, W - 1);
  const V3 d0 = load3(rays_d, p0), d7 = load3(rays_d, p7);
  float ux = d7.x - d0.x, uy = d7.y - d0.y, uz = d7.z - d0.z;
  if (!(ux * ux + uy * uy + uz * uz > 1e-12f)) {
    ux = fabsf(ax) < 0.57f ? 1.f : 0.f; uy = fabsf(ax) < 0.57f ? 0.f : 1.f; uz = 0.f;
  }
  const float ua = ux * ax + uy * ay + uz * az;
  ux -= ua * ax; uy -= ua * ay; uz -= ua * az;
  const float uinv = rsqrtf(ux * ux + uy * uy + uz * uz);
  ux *= uinv; uy *= uinv; uz *= uinv;
  const float vx = ay * uz - az * uy, vy = az * ux - ax * uz, vz = ax * uy - ay * ux;
  float a0 = 3e38f, a1 = -3e38f, b0 = 3e38f, b1 = -3e38f, cmin = 3e38f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float da = dd[h].x * ax + dd[h].y * ay + dd[h].z * az;
    const float al = (dd[h].x * ux + dd[h].y * uy + dd[h].z * uz) / da;
    const float be = (dd[h].x * vx + dd[h].y * vy + dd[h].z * vz) / da;
    const float len2 = dd[h].x * dd[h].x + dd[h].y * dd[h].y + dd[h].z * dd[h].z;
    cmin = fminf(cmin, da * rsqrtf(len2));
    same = same && (al == al) && (be == be) && fabsf(al) < 1e6f && fabsf(be) < 1e6f;
    a0 = fminf(a0, al); a1 = fmaxf(a1, al); b0 = fminf(b0, be); b1 = fmaxf(b1, be);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    a0 = fminf(a0, __shfl_xor_sync(0xffffffffu, a0, off)); a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, off));
    b0 = fminf(b0, __shfl_xor_sync(0xffffffffu, b0, off)); b1 = fmaxf(b1, __shfl_xor_sync(0xffffffffu, b1, off));
    cmin = fminf(cmin, __shfl_xor_sync(0xffffffffu, cmin, off));
  }
  same = __all_sync(0xffffffffu, same);
  const bool ok = same && cmin > 0.5f && (ax == ax) && (ux == ux) && fabsf(o0.x) < 1e30f && fabsf(o0.y) < 1e30f &&
                  fabsf(o0.z) < 1e30f;
  if (lane == 0) {
    TileFrame f;
    // inflate the rectangle: rounding of the coordinates themselves
    const float pa = 1e-5f + 1e-3f * (a1 - a0), pb = 1e-5f + 1e-3f * (b1 - b0);
    f.ox = o0.x; f.oy = o0.y; f.oz = o0.z; f.ax = ax; f.ay = ay; f.az = az;
    f.ux = ux; f.uy = uy; f.uz = uz; f.vx = vx; f.vy = vy; f.vz = vz;
    f.a0 = ok ? a0 - pa : 1.f; f.a1 = ok ? a1 + pa : -1.f;
    f.b0 = b0 - pb; f.b1 = b1 + pb;
    frames[tile] = f;
  }
}

void launch_tile_frames(const mlpsp_frame* fr, TileFrame* frames, cudaStream_t st) {
  const int T = num_tiles(fr->width, fr->height, 8);
  const int ntx = (fr->width + 7) / 8;
  k_tile_frames<<<(T + 7) / 8, 256, 0, st>>>(fr->rays_o, fr->rays_d, fr->width, fr->height, ntx, T, frames);
}

int launch_sort(const mlpsp_scene* sc, const mlpsp_frame* fr, float* keys_out, cudaStream_t st, bool unordered_input,
                int32_t* long_list, int32_t* long_count, const int32_t* list_len) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  const int ntx = (fr->width + fr->tile - 1) / fr->tile;
  MLPSP_REQUIRE(fr->tile_capacity > 0 && fr->tile_capacity <= kSortCap, MLPSP_E_LIMIT,
                "tile_capacity must be in [1, %d]", kSortCap);
  MLPSP_REQUIRE(long_list && long_count, MLPSP_E_ARG, "sort: scratch for the long-tile list missing");
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  MLPSP_CUDA_OK(cudaMemsetAsync(long_count, 0, 8, st));   // tile cursors: [0] of k_sort_long, [1] of k_sort_tiles
  LaunchScope scope(kKSort, 2, st);
  const int grid = std::min((T + kTilesPerCta - 1) / kTilesPerCta, sms * 6);
  const int grid_long = std::min(T, sms * 6);
  const float4* geom = (const float4*)sc->geom;
  // the reference kernels' arithmetic exists for the tile-centre key only (sort_key 0)
  const int key_mode = fr->sort_key | ((fr->hit_arith == 1 && fr->sort_key == 0) ? 4 : 0);
  if (unordered_input) {
    launch_chained(k_sort_long<256, kSortCap, true>, dim3(grid_long), dim3(256), 0, st, fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets,
                   fr->tile_prims, fr->width, fr->height, fr->tile, ntx, fr->sorted_prims, keys_out, key_mode, T, long_count, list_len, fr->status);
    launch_chained(k_sort_tiles<true>, dim3(grid), dim3(256), 0, st, fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets, fr->tile_prims,
                   fr->width, fr->height, fr->tile, ntx, T, kSortCap, fr->sorted_prims, keys_out, key_mode, long_list, long_count,
                   list_len, fr->status);
  } else {
    launch_chained(k_sort_long<256, kSortCap, false>, dim3(grid_long), dim3(256), 0, st, fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets,
                   fr->tile_prims, fr->width, fr->height, fr->tile, ntx, fr->sorted_prims, keys_out, key_mode, T, long_count, list_len, fr->status);
    launch_chained(k_sort_tiles<false>, dim3(grid), dim3(256), 0, st, fr->rays_o, fr->rays_d, geom, sc->n, fr->tile_offsets, fr->tile_prims,
                   fr->width, fr->height, fr->tile, ntx, T, kSortCap, fr->sorted_prims, keys_out, key_mode, long_list, long_count,
                   list_len, fr->status);
  }
  return cuda_check(cudaGetLastError(), "sort_tiles");
}

}  // namespace mlpsp
