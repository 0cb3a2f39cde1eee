// Geometry packing and screen-space tile binning.
//
// Binning restates the PyTorch culling of scannet/cumodel.py:994-1070 without the dense
// [tiles x primitives] matrix: one thread per primitive projects its bounding circle and derives
// the inclusive tile rectangle that satisfies the strict overlap predicate; a count pass, a scan
// over tiles and a scatter pass build the tile-major lists, and a per-tile radix sort by id puts
// every list in ascending primitive order (the order nonzero() gives the reference).
#include <algorithm>
#include "frame.cuh"
#include "block_sort.cuh"

namespace mlpsp {

// ------------------------------------------------------------------ packing / normalise ----
__global__ void k_pack_geometry(const float* __restrict__ pos, const float* __restrict__ ls,
                                const float* __restrict__ quat, int n, float4* __restrict__ geom) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float lx = ls[i * 3], ly = ls[i * 3 + 1], lz = ls[i * 3 + 2];
  const float sx = det_exp(lx), sy = det_exp(ly), sz = det_exp(lz);
  geom[(size_t)i * 4 + 0] = make_float4(pos[i * 3], pos[i * 3 + 1], pos[i * 3 + 2], quat[i * 4]);
  geom[(size_t)i * 4 + 1] = make_float4(quat[i * 4 + 1], quat[i * 4 + 2], quat[i * 4 + 3], fmaxf(fmaxf(sx, sy), sz));
  geom[(size_t)i * 4 + 2] = make_float4(det_exp(fmul(-2.f, lx)), det_exp(fmul(-2.f, ly)), det_exp(fmul(-2.f, lz)), 0.f);
  geom[(size_t)i * 4 + 3] = make_float4(lx, ly, lz, 0.f);
}

template <int DIM>
__global__ void k_normalize_rows(const float* __restrict__ in, float* __restrict__ out, int64_t rows) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  float a[DIM];
#pragma unroll
  for (int k = 0; k < DIM; ++k) a[k] = in[i * DIM + k];
  float s = fmul(a[0], a[0]);
#pragma unroll
  for (int k = 1; k < DIM; ++k) s = ffma(a[k], a[k], s);
  const float nrm = fmaxf(__fsqrt_rn(s), 1e-12f);
#pragma unroll
  for (int k = 0; k < DIM; ++k) out[i * DIM + k] = fdiv(a[k], nrm);
}

// ------------------------------------------------------------------------------ binning ----
struct BinCam {
  float view[16];
  float proj[16];
  float radius_mult, focal;
  int W, H, ts, ntx, nty;
  int row0, row1;   // tile rows kept: [row0, row1)
};

__device__ __forceinline__ float dot4(const float* row, float x, float y, float z, float w) {
  float a = fmul(row[0], x);
  a = ffma(row[1], y, a);
  a = ffma(row[2], z, a);
  a = ffma(row[3], w, a);
  return a;
}

// smallest t with (t+1)*ts > lo and largest t with t*ts < hi, clipped to [0, nt)
__device__ __forceinline__ bool tile_span(float lo, float hi, int ts, int nt, int& t0, int& t1) {
  if (!(lo == lo) || !(hi == hi)) return false;
  const float fts = (float)ts;
  int a, b;
  if (lo < 0.f) a = 0;
  else if (lo >= fmul((float)nt, fts)) return false;
  else {
    a = (int)fdiv(lo, fts);
    while (a > 0 && (float)(a * ts) > lo) --a;
    while ((float)((a + 1) * ts) <= lo) ++a;
  }
  if (hi <= 0.f) return false;
  else if (hi > fmul((float)(nt - 1), fts)) b = nt - 1;
  else {
    b = (int)fdiv(hi, fts);
    while ((float)(b * ts) >= hi) --b;
    while (b + 1 < nt && (float)((b + 1) * ts) < hi) ++b;
  }
  if (a >= nt || b < 0 || a > b) return false;
  t0 = a; t1 = b;
  return true;
}

__device__ __forceinline__ bool prim_rect(const float4* __restrict__ geom, int p, const BinCam& c, int r[4]) {
  const float4 g0 = __ldg(geom + (size_t)p * 4);
  const float smax = __ldg(geom + (size_t)p * 4 + 1).w;
  const float vx = dot4(c.view + 0, g0.x, g0.y, g0.z, 1.f);
  const float vy = dot4(c.view + 4, g0.x, g0.y, g0.z, 1.f);
  const float vz = dot4(c.view + 8, g0.x, g0.y, g0.z, 1.f);
  const float vw = dot4(c.view + 12, g0.x, g0.y, g0.z, 1.f);
  if (!(vz > 0.001f)) return false;
  const float world_r = fmul(smax, c.radius_mult);
  const float pix_r = fmul(fdiv(world_r, fadd(vz, 1e-8f)), c.focal);
  const float cx = dot4(c.proj + 0, vx, vy, vz, vw);
  const float cy = dot4(c.proj + 4, vx, vy, vz, vw);
  float cw = dot4(c.proj + 12, vx, vy, vz, vw);
  if (cw == 0.f) cw = fadd(cw, 1e-6f);
  const float nx = fdiv(cx, cw), ny = fdiv(cy, cw);
  const float sx = fmul(fmul(fadd(nx, 1.f), 0.5f), (float)c.W);
  const float sy = fmul(fmul(fadd(ny, 1.f), 0.5f), (float)c.H);
  if (!tile_span(fsub(sx, pix_r), fadd(sx, pix_r), c.ts, c.ntx, r[0], r[1])) return false;
  if (!tile_span(fsub(sy, pix_r), fadd(sy, pix_r), c.ts, c.nty, r[2], r[3])) return false;
  r[2] = max(r[2], c.row0);
  r[3] = min(r[3], c.row1 - 1);
  return r[2] <= r[3];
}

// Visit every tile of this thread's rectangle; rectangles larger than 32 tiles are walked by the
// whole warp so one near primitive cannot serialise a thread.
template <typename F>
__device__ __forceinline__ void for_each_tile(bool has, int x0, int x1, int y0, int y1, int ntx, int p, F f) {
  const int w = x1 - x0 + 1, h = y1 - y0 + 1;
  const int area = has ? w * h : 0;
  const bool big = area > 32;
  if (has && !big)
    for (int ty = y0; ty <= y1; ++ty)
      for (int tx = x0; tx <= x1; ++tx) f(ty * ntx + tx, p);
  unsigned bigs = __ballot_sync(0xffffffffu, big);
  const int lane = threadIdx.x & 31;
  while (bigs) {
    const int src = __ffs(bigs) - 1;
    bigs &= bigs - 1;
    const int bx0 = __shfl_sync(0xffffffffu, x0, src), by0 = __shfl_sync(0xffffffffu, y0, src);
    const int bw = __shfl_sync(0xffffffffu, w, src), ba = __shfl_sync(0xffffffffu, area, src);
    const int bp = __shfl_sync(0xffffffffu, p, src);
    for (int i = lane; i < ba; i += 32) f((by0 + i / bw) * ntx + bx0 + i % bw, bp);
  }
}

// Warp-flattened walk over the tiles of 32 rectangles.  Lane l brings rectangle l (none when !has); the
// rectangles' tiles form one list of `total` items that the lanes share evenly: item i belongs to the
// rectangle j with pref[j] <= i < pref[j + 1].  Iterations are independent, so the atomics of several
// of them are in flight at once, whatever the sizes of the individual rectangles.
struct WarpRects { int pref[33]; int x0[32], y0[32], w[32], p[32]; };
struct WarpWhiten { PrimWhiten w[8]; };   // whitening maps of a warp's primitives (pre-tested scatter)

template <typename F>
__device__ __forceinline__ void for_each_tile_flat(bool has, int x0, int x1, int y0, int y1, int ntx, int p,
                                                   WarpRects& wr, F f) {
  const int lane = threadIdx.x & 31;
  const int w = x1 - x0 + 1;
  const int area = has ? w * (y1 - y0 + 1) : 0;
  int inc = area;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += v;
  }
  const int total = __shfl_sync(0xffffffffu, inc, 31);
  if (lane == 0) wr.pref[0] = 0;
  wr.pref[lane + 1] = inc;
  wr.x0[lane] = x0; wr.y0[lane] = y0; wr.w[lane] = w; wr.p[lane] = p;
  __syncwarp();
#pragma unroll 4
  for (int i = lane; i < total; i += 32) {
    int j = 0;
#pragma unroll
    for (int step = 16; step > 0; step >>= 1)
      if (wr.pref[j + step] <= i) j += step;
    const int k = i - wr.pref[j], bw = wr.w[j];
    const int row = k / bw;
    f((wr.y0[j] + row) * ntx + wr.x0[j] + (k - row * bw), wr.p[j]);
  }
  __syncwarp();
}

__global__ void __launch_bounds__(256) k_bin_count(const float4* __restrict__ geom, int n, BinCam cam,
                                                   uint2* __restrict__ rect, int32_t* __restrict__ tile_cnt) {
  chain_wait();
  chain_release();
  __shared__ WarpRects s_wr[8];
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  int r[4] = {1, 0, 1, 0};
  const bool has = (p < n) && prim_rect(geom, p, cam, r);
  if (p < n) rect[p] = has ? make_uint2((uint32_t)r[0] | ((uint32_t)r[1] << 16), (uint32_t)r[2] | ((uint32_t)r[3] << 16))
                           : make_uint2(1u, 1u);  // x0=1 > x1=0
  for_each_tile_flat(has, r[0], r[1], r[2], r[3], cam.ntx, p, s_wr[threadIdx.x >> 5],
                     [&](int t, int) { atomicAdd(tile_cnt + t, 1); });
}

// The count pass without a walk over the tiles: a rectangle adds its four corners to a 2-D difference array
// (+1, -1, -1, +1), and the 2-D prefix sum of that array is the number of rectangles over each tile.  Four atomics
// per primitive instead of one per (tile, primitive) pair (100,000 against 2.9 million on the bench frame).
__global__ void __launch_bounds__(256) k_bin_corners(const float4* __restrict__ geom, int n, BinCam cam,
                                                     uint2* __restrict__ rect, int32_t* __restrict__ diff) {
  chain_wait();
  chain_release();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  int r[4] = {1, 0, 1, 0};
  const bool has = prim_rect(geom, p, cam, r);
  rect[p] = has ? make_uint2((uint32_t)r[0] | ((uint32_t)r[1] << 16), (uint32_t)r[2] | ((uint32_t)r[3] << 16))
                : make_uint2(1u, 1u);  // x0=1 > x1=0
  if (has) {
    const int sx = cam.ntx + 1;
    atomicAdd(diff + r[2] * sx + r[0], 1);
    atomicAdd(diff + r[2] * sx + r[1] + 1, -1);
    atomicAdd(diff + (r[3] + 1) * sx + r[0], -1);
    atomicAdd(diff + (r[3] + 1) * sx + r[1] + 1, 1);
  }
}

// One CTA turns the corner array into the tile offsets: prefix sums along the rows and then along the columns (in
// shared memory) give the per-tile counts; their exclusive prefix in tile order is tile_offsets; the longest list,
// the capacity check and the pair total of k_bin_finish ride along.
__global__ void __launch_bounds__(1024) k_bin_offsets(const int32_t* __restrict__ diff, int ntx, int nty,
                                                      int32_t* __restrict__ tile_offsets, int capacity, int64_t max_pairs,
                                                      int32_t* __restrict__ status, int32_t* __restrict__ counters) {
  extern __shared__ int32_t s_cnt[];          // [(nty + 1)][(ntx + 1)]
  __shared__ int warp_sums[32];
  chain_wait();
  chain_release();
  const int sx = ntx + 1, T = ntx * nty, tid = threadIdx.x;
  for (int i = tid; i < sx * (nty + 1); i += 1024) s_cnt[i] = diff[i];
  __syncthreads();
  for (int y = tid; y < nty; y += 1024) {
    int acc = 0;
    for (int x = 0; x < ntx; ++x) { acc += s_cnt[y * sx + x]; s_cnt[y * sx + x] = acc; }
  }
  __syncthreads();
  for (int x = tid; x < ntx; x += 1024) {
    int acc = 0;
    for (int y = 0; y < nty; ++y) { acc += s_cnt[y * sx + x]; s_cnt[y * sx + x] = acc; }
  }
  __syncthreads();
  const int per = (T + 1023) / 1024;
  const int b = min(T, tid * per), e = min(T, b + per);
  int sum = 0, mx = 0;
  for (int t = b; t < e; ++t) {
    const int c = s_cnt[(t / ntx) * sx + t % ntx];
    sum += c;
    mx = max(mx, c);
  }
  int total;
  int ex = block_exclusive_scan(sum, warp_sums, total);
  for (int t = b; t < e; ++t) { tile_offsets[t] = ex; ex += s_cnt[(t / ntx) * sx + t % ntx]; }
  mx = __reduce_max_sync(0xffffffffu, mx);
  if ((tid & 31) == 0 && mx > 0) {
    atomicMax(status + MLPSP_ST_MAX_TILE_LEN, mx);
    if (capacity > 0 && mx > capacity) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TILE_CAPACITY);
  }
  if (tid == 0) {
    tile_offsets[T] = total;
    status[MLPSP_ST_PAIRS] = total;
    counters[kCtrPairs] = total;
    if (total < 0 || (int64_t)total > max_pairs) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_PAIR_OVERFLOW);
  }
}

// PRETEST: a (tile, primitive) pair that no ray of the tile can hit (tile_surely_misses) is not
// written; tile_fill then ends as the number of candidates kept per tile, packed at the front of the
// tile's span of tile_prims (the span itself keeps the size the count pass gave it).
// PPW primitives per warp: the pre-tested variant does a few hundred instructions and three dependent memory
// round trips per pair, so it spreads the pairs over four times as many warps.
template <bool PRETEST, int PPW>
__global__ void __launch_bounds__(256) k_bin_scatter(int n, int ntx, const uint2* __restrict__ rect,
                                                     const int32_t* __restrict__ tile_offsets,
                                                     int32_t* __restrict__ tile_fill, int32_t* __restrict__ tile_prims,
                                                     const float4* __restrict__ geom,
                                                     const TileFrame* __restrict__ frames, float K0,
                                                     const int32_t* __restrict__ status) {
  chain_wait();
  chain_release();
  __shared__ WarpRects s_wr[8];
  __shared__ WarpWhiten s_ww[PRETEST ? 8 : 1];
  static_assert(!PRETEST || PPW <= 8, "WarpWhiten holds eight maps per warp");
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * 8 + warp;
  const int p = gwarp * PPW + lane;
  int x0 = 1, x1 = 0, y0 = 1, y1 = 0;
  const bool mine = lane < PPW && p < n;
  if (mine) {
    const uint2 r = rect[p];
    x0 = r.x & 0xffff; x1 = r.x >> 16; y0 = r.y & 0xffff; y1 = r.y >> 16;
  }
  const bool has = mine && x0 <= x1 && y0 <= y1;
  if (PRETEST && has) s_ww[warp].w[lane] = make_whiten(load_geom(geom, p));
  // (for_each_tile_flat synchronises the warp before the first item is read)
  for_each_tile_flat(has, x0, x1, y0, y1, ntx, PRETEST ? lane : p, s_wr[warp], [&](int t, int q) {
    int id = q;
    if (PRETEST) {
      // q is the lane that brought the primitive: its map sits in shared memory
      const float4* fp = reinterpret_cast<const float4*>(frames + t);
      const float4 f0 = __ldg(fp), f1 = __ldg(fp + 1), f2 = __ldg(fp + 2), f3 = __ldg(fp + 3);
      const TileFrame f = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w, f2.x, f2.y, f2.z, f2.w, f3.x, f3.y, f3.z, f3.w};
      if (tile_surely_misses(s_ww[warp].w[q], f, K0)) return;
      id = gwarp * PPW + q;
    }
    const int slot = atomicAdd(tile_fill + t, 1);
    tile_prims[tile_offsets[t] + slot] = id;
  });
}

// Mosaic frames: every tile is drawn from one of K views (build_tilecenter_culling_from_tile_views,
// scannet/cumodel.py:838-949).  blockIdx.y selects the view; a primitive's rectangle under that view
// contributes only the tiles assigned to it.
constexpr int kViewBatch = 8;
struct BinCams { BinCam cam[kViewBatch]; };

template <bool SCATTER>
__global__ void k_bin_views(const float4* __restrict__ geom, int n, BinCams cams, int view0,
                            const int32_t* __restrict__ tile_view, int32_t* __restrict__ tile_cnt,
                            const int32_t* __restrict__ tile_offsets, int32_t* __restrict__ tile_prims,
                            const int32_t* __restrict__ status) {
  if (SCATTER && (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL)) return;
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  const BinCam& cam = cams.cam[blockIdx.y];
  const int view = view0 + blockIdx.y;
  int r[4] = {1, 0, 1, 0};
  const bool has = (p < n) && prim_rect(geom, p, cam, r);
  for_each_tile(has, r[0], r[1], r[2], r[3], cam.ntx, p, [&](int t, int q) {
    if (tile_view[t] != view) return;
    if (SCATTER) tile_prims[tile_offsets[t] + atomicAdd(tile_cnt + t, 1)] = q;
    else atomicAdd(tile_cnt + t, 1);
  });
}

// ------------------------------------------------------------- multi-block exclusive scan ----
__global__ void k_scan_partial(const int32_t* __restrict__ in, int64_t n, int32_t* __restrict__ blk) {
  chain_wait();
  chain_release();
  __shared__ int warp_sums[32];
  const int64_t base = (int64_t)blockIdx.x * kScanItems;
  int v = 0;
  for (int j = 0; j < kScanItems / 1024; ++j) {
    const int64_t i = base + threadIdx.x + j * 1024;
    if (i < n) v += in[i];
  }
  int total;
  block_exclusive_scan(v, warp_sums, total);
  if (threadIdx.x == 0) blk[blockIdx.x] = total;
}

// single block: exclusive scan of blk[0,nblk) in place, grand total -> blk[nblk]
__global__ void k_scan_top(int32_t* __restrict__ blk, int nblk) {
  chain_wait();
  chain_release();
  __shared__ int warp_sums[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nblk; b0 += 1024) {
    const int i = b0 + threadIdx.x;
    const int v = (i < nblk) ? blk[i] : 0;
    int total;
    const int ex = block_exclusive_scan(v, warp_sums, total);
    const int c = carry;
    if (i < nblk) blk[i] = c + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry = c + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) blk[nblk] = carry;
}

// out[i] = exclusive prefix; out[n] = total.  Thread t of a block owns 4 consecutive items.
__global__ void k_scan_final(const int32_t* __restrict__ in, int64_t n, const int32_t* __restrict__ blk,
                             int32_t* __restrict__ out) {
  chain_wait();
  chain_release();
  __shared__ int warp_sums[32];
  const int64_t base = (int64_t)blockIdx.x * kScanItems + (int64_t)threadIdx.x * 4;
  int v[4], s = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = (base + j < n) ? in[base + j] : 0; s += v[j]; }
  int total;
  int ex = block_exclusive_scan(s, warp_sums, total) + blk[blockIdx.x];
#pragma unroll
  for (int j = 0; j < 4; ++j) { if (base + j < n) out[base + j] = ex; ex += v[j]; }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) out[n] = blk[gridDim.x];
}

// longest tile list, capacity check, pair total
__global__ void k_bin_finish(const int32_t* __restrict__ tile_cnt, int T, const int32_t* __restrict__ tile_offsets,
                             int capacity, int64_t max_pairs, int32_t* __restrict__ status,
                             int32_t* __restrict__ counters) {
  chain_wait();
  chain_release();
  int mx = 0;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) mx = max(mx, tile_cnt[t]);
  mx = __reduce_max_sync(0xffffffffu, mx);
  if ((threadIdx.x & 31) == 0 && mx > 0) {
    atomicMax(status + MLPSP_ST_MAX_TILE_LEN, mx);
    if (capacity > 0 && mx > capacity) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TILE_CAPACITY);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const int M = tile_offsets[T];
    status[MLPSP_ST_PAIRS] = M;
    counters[kCtrPairs] = M;
    if (M < 0 || (int64_t)M > max_pairs) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_PAIR_OVERFLOW);
  }
}

// per-tile ascending sort of candidate ids (lists no longer than CAP; longer lists were rejected)
template <int THREADS, int CAP>
__global__ void __launch_bounds__(THREADS) k_sort_ids(const int32_t* __restrict__ tile_offsets,
                                                      int32_t* __restrict__ tile_prims,
                                                      const int32_t* __restrict__ status) {
  using Sort = BlockRadixSort<THREADS, CAP>;
  __shared__ typename Sort::Smem sm;
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int s = tile_offsets[blockIdx.x], e = tile_offsets[blockIdx.x + 1];
  const int n = min(e - s, CAP);
  if (n <= 1) return;
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const int32_t p = tile_prims[s + i];
    sm.key[0][i] = (uint32_t)p;
    sm.val[0][i] = p;
  }
  __syncthreads();
  const int cur = Sort::sort(sm, n);
  for (int i = threadIdx.x; i < n; i += THREADS) tile_prims[s + i] = sm.val[cur][i];
}

// The same scan by one CTA for inputs of at most 32,768 items (the tile counts of a frame up to 1920x1080):
// thread t owns the items [t * per, t * per + per).  One launch instead of three.
constexpr int kScanSmallMax = 32768;
__global__ void __launch_bounds__(1024) k_scan_small(const int32_t* __restrict__ in, int n, int32_t* __restrict__ out) {
  chain_wait();
  chain_release();
  __shared__ int warp_sums[32];
  const int per = (n + 1023) / 1024;
  const int b = min(n, (int)threadIdx.x * per), e = min(n, b + per);
  int s = 0;
  for (int i = b; i < e; ++i) s += in[i];
  int total;
  int ex = block_exclusive_scan(s, warp_sums, total);
  for (int i = b; i < e; ++i) { const int v = in[i]; out[i] = ex; ex += v; }
  if (threadIdx.x == 0) out[n] = total;
}

int scan_launches(int64_t n) { return n <= 0 ? 0 : (n <= kScanSmallMax ? 1 : 3); }

int launch_scan_i32(const int32_t* in, int64_t n, int32_t* blk, int32_t* out, cudaStream_t st) {
  const int nblk = (int)((n + kScanItems - 1) / kScanItems);
  if (nblk == 0) return MLPSP_OK;
  if (n <= kScanSmallMax && in != out) {
    launch_chained(k_scan_small, dim3(1), dim3(1024), 0, st, in, (int)n, out);
    return cuda_check(cudaGetLastError(), "scan");
  }
  launch_chained(k_scan_partial, dim3(nblk), dim3(1024), 0, st, in, n, blk);
  launch_chained(k_scan_top, dim3(1), dim3(1024), 0, st, blk, nblk);
  launch_chained(k_scan_final, dim3(nblk), dim3(1024), 0, st, in, n, blk, out);
  return cuda_check(cudaGetLastError(), "scan");
}

constexpr int kSortCap = 2048;  // per-tile sort capacity (>= tile capacity 1536)

int launch_bin(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st, bool order_lists,
               bool pretest) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  BinCam cam;
  for (int i = 0; i < 16; ++i) { cam.view[i] = fr->view[i]; cam.proj[i] = fr->proj[i]; }
  cam.radius_mult = (float)sqrt(-2.0 * log((double)fr->threshold));
  const float fx = (cam.proj[0] * (float)fr->width) / 2.0f;
  const float fy = (cam.proj[5] * (float)fr->height) / 2.0f;
  cam.focal = (fx + fy) * 0.5f;
  cam.W = fr->width; cam.H = fr->height; cam.ts = fr->tile;
  cam.ntx = (fr->width + fr->tile - 1) / fr->tile;
  cam.nty = (fr->height + fr->tile - 1) / fr->tile;
  cam.row0 = 0; cam.row1 = cam.nty;
  if (fr->tile_row_begin != 0 || fr->tile_row_end != 0) {
    MLPSP_REQUIRE(fr->tile_row_begin >= 0 && fr->tile_row_begin <= fr->tile_row_end && fr->tile_row_end <= cam.nty,
                  MLPSP_E_ARG, "tile row band [%d,%d) outside [0,%d]", fr->tile_row_begin, fr->tile_row_end, cam.nty);
    cam.row0 = fr->tile_row_begin; cam.row1 = fr->tile_row_end;
  }
  MLPSP_REQUIRE(cam.ntx < 65536 && cam.nty < 65536, MLPSP_E_LIMIT, "tile grid beyond 65535 per axis");
  MLPSP_REQUIRE(fr->tile_capacity > 0 && fr->tile_capacity <= kSortCap, MLPSP_E_LIMIT,
                "tile_capacity must be in [1, %d]", kSortCap);
  MLPSP_REQUIRE(!(pretest && order_lists), MLPSP_E_ARG, "bin: the tile pre-test leaves the lists in scatter order");
  MLPSP_REQUIRE(!pretest || (fr->tile == 8 && fr->rays_o && fr->rays_d), MLPSP_E_ARG,
                "bin: the tile pre-test needs 8x8 tiles and the frame's rays");
  // with the pre-test the per-tile fill counters are the traversal lengths the wave kernels read
  int32_t* fill = pretest ? s.tile_len : s.tile_fill;
  const int n = sc->n;
  // count pass: rectangle corners + one CTA's 2-D prefix when the corner array fits its shared memory (frames up
  // to about 3,500 x 3,500 pixels), else one atomic per (tile, primitive) pair and the multi-block scan
  const size_t diff_bytes = 4 * (size_t)(cam.ntx + 1) * (cam.nty + 1);
  const bool corners = diff_bytes <= 200 * 1024;
  if (corners) MLPSP_CUDA_OK(cudaMemsetAsync(s.tile_diff, 0, diff_bytes, st));
  else MLPSP_CUDA_OK(cudaMemsetAsync(s.tile_cnt, 0, 4 * (size_t)(T + 1), st));
  MLPSP_CUDA_OK(cudaMemsetAsync(fill, 0, 4 * (size_t)T, st));
  LaunchScope scope(kKBin, (n > 0 ? (order_lists ? 3 : 2) : 0) + (corners ? 1 : 1 + scan_launches(T)) + (pretest ? 1 : 0), st);
  if (pretest) launch_tile_frames(fr, s.tile_frame, st);
  if (corners) {
    static DeviceOnce attr_once;
    if (attr_once.first())
      MLPSP_CUDA_OK(cudaFuncSetAttribute(k_bin_offsets, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    if (n > 0) launch_chained(k_bin_corners, dim3((n + 255) / 256), dim3(256), 0, st, (const float4*)sc->geom, n, cam, s.rect, s.tile_diff);
    launch_chained(k_bin_offsets, dim3(1), dim3(1024), diff_bytes, st, s.tile_diff, cam.ntx, cam.nty, fr->tile_offsets, fr->tile_capacity,
                   fr->max_pairs, fr->status, s.counters);
  } else {
    if (n > 0) launch_chained(k_bin_count, dim3((n + 255) / 256), dim3(256), 0, st, (const float4*)sc->geom, n, cam, s.rect, s.tile_cnt);
    int rc = launch_scan_i32(s.tile_cnt, T, s.scan_blk, fr->tile_offsets, st);
    if (rc) return rc;
    launch_chained(k_bin_finish, dim3(std::min(64, (T + 255) / 256)), dim3(256), 0, st, s.tile_cnt, T, fr->tile_offsets, fr->tile_capacity,
                   fr->max_pairs, fr->status, s.counters);
  }
  if (n > 0) {
    if (pretest)
      launch_chained(k_bin_scatter<true, 8>, dim3((n + 63) / 64), dim3(256), 0, st, n, cam.ntx, s.rect, fr->tile_offsets, fill, fr->tile_prims,
                                                           (const float4*)sc->geom, s.tile_frame,
                                                           (float)(-2.0 * log((double)fr->threshold)), fr->status);
    else
      launch_chained(k_bin_scatter<false, 32>, dim3((n + 255) / 256), dim3(256), 0, st, n, cam.ntx, s.rect, fr->tile_offsets, fill, fr->tile_prims,
                                                            nullptr, nullptr, 0.f, fr->status);
    if (order_lists) k_sort_ids<256, kSortCap><<<T, 256, 0, st>>>(fr->tile_offsets, fr->tile_prims, fr->status);
  }
  return cuda_check(cudaGetLastError(), "bin");
}

// ------------------------------------------------------------------- ray-cone culling ----
// scannet/camera.py:102-146.  One thread per tile builds the cone of the tile's 64 rays (pixel
// coordinates clamped to the image, sums in pixel order); one thread per primitive then walks a
// chunk of tiles whose cones sit in shared memory.
struct Cone { float ox, oy, oz, ax, ay, az, cos_t, sin_t; };

__device__ __forceinline__ void normalize3(float x, float y, float z, float& nx, float& ny, float& nz) {
  const float s = ffma(z, z, ffma(y, y, fmul(x, x)));
  const float nrm = fmaxf(__fsqrt_rn(s), 1e-12f);
  nx = fdiv(x, nrm); ny = fdiv(y, nrm); nz = fdiv(z, nrm);
}

__global__ void k_tile_cones(const float* __restrict__ rays_o, const float* __restrict__ rays_d, int W, int H, int ntx,
                             int T, Cone* __restrict__ cones, int32_t* __restrict__ status) {
  const int tile = blockIdx.x * blockDim.x + threadIdx.x;
  if (tile >= T) return;
  const int tx = tile % ntx, ty = tile / ntx;
  float sx = 0.f, sy = 0.f, sz = 0.f;
  const int64_t p0 = (int64_t)min(ty * 8, H - 1) * W + min(tx * 8, W - 1);
  const V3 o0 = load3(rays_o, p0);
  bool bad_origin = false;
  for (int k = 0; k < 64; ++k) {
    const int64_t pix = (int64_t)min(ty * 8 + (k >> 3), H - 1) * W + min(tx * 8 + (k & 7), W - 1);
    const V3 o = load3(rays_o, pix), d = load3(rays_d, pix);
    bad_origin |= fabsf(fsub(o.x, o0.x)) > 1e-6f || fabsf(fsub(o.y, o0.y)) > 1e-6f || fabsf(fsub(o.z, o0.z)) > 1e-6f;
    float nx, ny, nz;
    normalize3(d.x, d.y, d.z, nx, ny, nz);
    sx = fadd(sx, nx); sy = fadd(sy, ny); sz = fadd(sz, nz);
  }
  float ax, ay, az;
  normalize3(fdiv(sx, 64.f), fdiv(sy, 64.f), fdiv(sz, 64.f), ax, ay, az);
  float cmin = 2.f;
  for (int k = 0; k < 64; ++k) {
    const int64_t pix = (int64_t)min(ty * 8 + (k >> 3), H - 1) * W + min(tx * 8 + (k & 7), W - 1);
    const V3 d = load3(rays_d, pix);
    float nx, ny, nz;
    normalize3(d.x, d.y, d.z, nx, ny, nz);
    cmin = fminf(cmin, ffma(nz, az, ffma(ny, ay, fmul(nx, ax))));
  }
  cmin = fminf(1.f, fmaxf(-1.f, cmin));
  Cone c;
  c.ox = o0.x; c.oy = o0.y; c.oz = o0.z; c.ax = ax; c.ay = ay; c.az = az; c.cos_t = cmin;
  c.sin_t = __fsqrt_rn(fmaxf(fsub(1.f, fmul(cmin, cmin)), 0.f));
  cones[tile] = c;
  if (bad_origin) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TILE_ORIGINS);
  if (!(cmin > 0.f)) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_CONE_TOO_WIDE);
}

__device__ __forceinline__ bool cone_keeps(const Cone& c, float px, float py, float pz, float radius) {
  const float dx = fsub(px, c.ox), dy = fsub(py, c.oy), dz = fsub(pz, c.oz);
  const float dist = __fsqrt_rn(ffma(dz, dz, ffma(dy, dy, fmul(dx, dx))));
  const float dc = fmaxf(dist, 1e-20f);
  const float ratio = fminf(1.f, fmaxf(0.f, fdiv(radius, dc)));
  const float cos_b = fdiv(ffma(dz, c.az, ffma(dy, c.ay, fmul(dx, c.ax))), dc);
  const float bound = fsub(fmul(c.cos_t, __fsqrt_rn(fmaxf(fsub(1.f, fmul(ratio, ratio)), 0.f))), fmul(c.sin_t, ratio));
  return (dist <= radius) || (cos_b >= fsub(bound, 2e-6f));
}

constexpr int kConeChunk = 128;   // tiles per block, as the reference's tile_chunk

template <bool SCATTER>
__global__ void __launch_bounds__(256) k_cone_bin(const float4* __restrict__ geom, int n, const Cone* __restrict__ cones,
                                                  int T, float radius_mult, int32_t* __restrict__ tile_cnt,
                                                  const int32_t* __restrict__ tile_offsets,
                                                  int32_t* __restrict__ tile_prims, const int32_t* __restrict__ status) {
  __shared__ Cone s_cone[kConeChunk];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int t0 = blockIdx.y * kConeChunk, nt = min(kConeChunk, T - t0);
  for (int i = threadIdx.x; i < nt; i += 256) s_cone[i] = cones[t0 + i];
  __syncthreads();
  const int p = blockIdx.x * 256 + threadIdx.x;
  float px = 0.f, py = 0.f, pz = 0.f, radius = -1.f;
  if (p < n) {
    const float4 g0 = __ldg(geom + (size_t)p * 4);
    px = g0.x; py = g0.y; pz = g0.z;
    radius = fadd(fmul(fmul(__ldg(geom + (size_t)p * 4 + 1).w, radius_mult), 1.00001f), 1e-7f);
  }
  const int lane = threadIdx.x & 31;
  for (int i = 0; i < nt; ++i) {
    const bool keep = (p < n) && cone_keeps(s_cone[i], px, py, pz, radius);
    const uint32_t m = __ballot_sync(0xffffffffu, keep);
    if (m == 0u) continue;
    int base = 0;
    if (lane == 0) base = atomicAdd(tile_cnt + t0 + i, __popc(m));
    if (SCATTER) {
      base = __shfl_sync(0xffffffffu, base, 0);
      if (keep) tile_prims[tile_offsets[t0 + i] + base + __popc(m & ((1u << lane) - 1u))] = p;
    }
  }
}

int launch_bin_raycone(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  const int ntx = (fr->width + 7) / 8;
  MLPSP_REQUIRE(fr->tile_capacity > 0 && fr->tile_capacity <= kSortCap, MLPSP_E_LIMIT,
                "tile_capacity must be in [1, %d]", kSortCap);
  MLPSP_REQUIRE(sizeof(Cone) * (size_t)T <= 16 * (size_t)fr->width * fr->height, MLPSP_E_LIMIT, "cone scratch too small");
  Cone* cones = reinterpret_cast<Cone*>(s.px_state);   // 32 B per tile inside the 16 B per pixel state array
  const float rm = (float)sqrt(-2.0 * log((double)fr->threshold));
  const int n = sc->n;
  MLPSP_CUDA_OK(cudaMemsetAsync(s.tile_cnt, 0, 4 * (size_t)(T + 1), st));
  MLPSP_CUDA_OK(cudaMemsetAsync(s.tile_fill, 0, 4 * (size_t)T, st));
  LaunchScope scope(kKBin, 5 + scan_launches(T), st);
  k_tile_cones<<<(T + 127) / 128, 128, 0, st>>>(fr->rays_o, fr->rays_d, fr->width, fr->height, ntx, T, cones, fr->status);
  const dim3 grid((std::max(n, 1) + 255) / 256, (T + kConeChunk - 1) / kConeChunk);
  if (n > 0) k_cone_bin<false><<<grid, 256, 0, st>>>((const float4*)sc->geom, n, cones, T, rm, s.tile_cnt, nullptr, nullptr, fr->status);
  int rc = launch_scan_i32(s.tile_cnt, T, s.scan_blk, fr->tile_offsets, st);
  if (rc) return rc;
  launch_chained(k_bin_finish, dim3(std::min(64, (T + 255) / 256)), dim3(256), 0, st, s.tile_cnt, T, fr->tile_offsets, fr->tile_capacity,
                                                              fr->max_pairs, fr->status, s.counters);
  if (n > 0) {
    k_cone_bin<true><<<grid, 256, 0, st>>>((const float4*)sc->geom, n, cones, T, rm, s.tile_fill, fr->tile_offsets,
                                           fr->tile_prims, fr->status);
    k_sort_ids<256, kSortCap><<<T, 256, 0, st>>>(fr->tile_offsets, fr->tile_prims, fr->status);
  }
  return cuda_check(cudaGetLastError(), "bin_raycone");
}

static BinCam make_cam(const mlpsp_frame* fr, const float* view) {
  BinCam cam;
  for (int i = 0; i < 16; ++i) { cam.view[i] = view[i]; cam.proj[i] = fr->proj[i]; }
  cam.radius_mult = (float)sqrt(-2.0 * log((double)fr->threshold));
  const float fx = (cam.proj[0] * (float)fr->width) / 2.0f;
  const float fy = (cam.proj[5] * (float)fr->height) / 2.0f;
  cam.focal = (fx + fy) * 0.5f;
  cam.W = fr->width; cam.H = fr->height; cam.ts = fr->tile;
  cam.ntx = (fr->width + fr->tile - 1) / fr->tile;
  cam.nty = (fr->height + fr->tile - 1) / fr->tile;
  cam.row0 = 0; cam.row1 = cam.nty;
  return cam;
}

int launch_bin_mosaic(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, const int32_t* tile_view,
                      const float* views_host, int num_views, cudaStream_t st) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  MLPSP_REQUIRE(fr->tile_capacity > 0 && fr->tile_capacity <= kSortCap, MLPSP_E_LIMIT,
                "tile_capacity must be in [1, %d]", kSortCap);
  MLPSP_CUDA_OK(cudaMemsetAsync(s.tile_cnt, 0, 4 * (size_t)(T + 1), st));
  MLPSP_CUDA_OK(cudaMemsetAsync(s.tile_fill, 0, 4 * (size_t)T, st));
  const int n = sc->n;
  const int batches = (num_views + kViewBatch - 1) / kViewBatch;
  LaunchScope scope(kKBin, 2 * batches + 2 + scan_launches(T), st);
  auto pass = [&](bool scatter) {
    for (int v0 = 0; v0 < num_views && n > 0; v0 += kViewBatch) {
      BinCams cams;
      const int nv = std::min(kViewBatch, num_views - v0);
      for (int v = 0; v < nv; ++v) cams.cam[v] = make_cam(fr, views_host + 16 * (size_t)(v0 + v));
      const dim3 grid((n + 255) / 256, nv);
      if (scatter)
        k_bin_views<true><<<grid, 256, 0, st>>>((const float4*)sc->geom, n, cams, v0, tile_view, s.tile_fill,
                                                fr->tile_offsets, fr->tile_prims, fr->status);
      else
        k_bin_views<false><<<grid, 256, 0, st>>>((const float4*)sc->geom, n, cams, v0, tile_view, s.tile_cnt,
                                                 fr->tile_offsets, fr->tile_prims, fr->status);
    }
  };
  pass(false);
  int rc = launch_scan_i32(s.tile_cnt, T, s.scan_blk, fr->tile_offsets, st);
  if (rc) return rc;
  launch_chained(k_bin_finish, dim3(std::min(64, (T + 255) / 256)), dim3(256), 0, st, s.tile_cnt, T, fr->tile_offsets, fr->tile_capacity,
                                                              fr->max_pairs, fr->status, s.counters);
  pass(true);
  if (n > 0) k_sort_ids<256, kSortCap><<<T, 256, 0, st>>>(fr->tile_offsets, fr->tile_prims, fr->status);
  return cuda_check(cudaGetLastError(), "bin_mosaic");
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int mlpsp_pack_geometry(const float* positions, const float* log_scales, const float* quats_unit,
                                   int32_t n, float* geom, void* stream) {
  MLPSP_REQUIRE(n >= 0 && (n == 0 || (positions && log_scales && quats_unit && geom)), MLPSP_E_ARG,
                "mlpsp_pack_geometry: null pointer or negative count");
  if (n == 0) return MLPSP_OK;
  LaunchScope scope(kKMisc, 1, (cudaStream_t)stream);
  k_pack_geometry<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(positions, log_scales, quats_unit, n, (float4*)geom);
  return cuda_check(cudaGetLastError(), "pack_geometry");
}

extern "C" int mlpsp_normalize_rows(const float* in, float* out, int64_t rows, int32_t dim, void* stream) {
  MLPSP_REQUIRE(rows >= 0 && (dim == 3 || dim == 4) && (rows == 0 || (in && out)), MLPSP_E_ARG,
                "mlpsp_normalize_rows: dim must be 3 or 4 and pointers non-null");
  if (rows == 0) return MLPSP_OK;
  const unsigned blocks = (unsigned)((rows + 255) / 256);
  LaunchScope scope(kKMisc, 1, (cudaStream_t)stream);
  if (dim == 3) k_normalize_rows<3><<<blocks, 256, 0, (cudaStream_t)stream>>>(in, out, rows);
  else k_normalize_rows<4><<<blocks, 256, 0, (cudaStream_t)stream>>>(in, out, rows);
  return cuda_check(cudaGetLastError(), "normalize_rows");
}
