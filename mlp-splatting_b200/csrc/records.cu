// Hit masks, primitive-major record construction (CSR), and front-to-back compositing.
//
// The reference walks a tile's sorted list serially and evaluates the MLP inside that walk
// (scannet/cuda/np_tile_kernels.cu:2110-2117).  Here the walk is cut into waves of consecutive
// list positions.  Per wave:
//   k_hits       every still-active pixel is tested against the wave's candidates
//                (hit_and_features_rot, np_tile_kernels.cu:659-711); one 64-bit mask per
//                (tile, candidate) pair, record slots reserved tile-major
//   prim scan    per-primitive record counts -> CSR offsets + evaluator work items
//   k_fill       (pixel, primitive) records written primitive-major: the 6-vector fed to the
//                encoder, decay, and the slot compositing will read
//   evaluator    per-primitive MLP over its records (mlp_f32.cu / mlp_tc.cu)
//   k_composite  per pixel, in list order, only while transmittance >= 1e-3
//                (np_tile_kernels.cu:2025-2136); tiles with a live pixel and candidates left go
//                on the next wave's list
// A record evaluated in a wave but reached after its pixel terminated inside the same wave is
// skipped by compositing, so results do not depend on the wave schedule.
#include <algorithm>
#include <climits>
#include <cmath>
#include "frame.cuh"

namespace mlpsp {

constexpr int kWinMax = 2048;

// squared bounding radius in units of the largest scale, with the 2 % margin surely_misses() relies on
static inline float miss_bound2(float thr) { return (float)(-2.0 * log((double)thr) * 1.02); }

// -------------------------------------------------------------------------- frame init ----
// One launch prepares a frame: pixel state and the output image, the list of live tiles and the wave counters,
// and the per-primitive counts and cursors of the first wave.
// tile_len (when not already written by the sort's tile pre-test) = the length of the caller's list.
__global__ void k_init_frame(int64_t P, float4* __restrict__ px_state, float2* __restrict__ px_depth,
                             float* __restrict__ rgb, float* __restrict__ alpha, float* __restrict__ depth_t,
                             float bgr, float bgg, float bgb, int T, int32_t* __restrict__ active0,
                             int32_t* __restrict__ counters, const int32_t* __restrict__ tile_offsets,
                             int32_t* __restrict__ tile_len, int lists_refined, int n, int32_t* __restrict__ prim_cnt,
                             int32_t* __restrict__ prim_cursor) {
  chain_wait();
  chain_release();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < P) {
    px_state[i] = make_float4(0.f, 0.f, 0.f, 1.f);
    px_depth[i] = make_float2(0.f, 0.f);
    rgb[i * 3] = bgr; rgb[i * 3 + 1] = bgg; rgb[i * 3 + 2] = bgb;
    alpha[i] = 0.f;
    if (depth_t) depth_t[i] = 0.f;
  }
  if (i < T) {
    active0[i] = (int)i;
    if (!lists_refined) tile_len[i] = tile_offsets[i + 1] - tile_offsets[i];
  }
  if (i < n) { prim_cnt[i] = 0; prim_cnt[prim_cnt_stride(n) + i] = 0; prim_cursor[i] = 0; }   // the counts of even and odd waves
  if (i == 0) {
    counters[kCtrRecords] = 0; counters[kCtrWork] = 0; counters[kCtrWorkNext] = 0; counters[kCtrWorkSmall] = 0;
    counters[kCtrActive0] = T; counters[kCtrActive1] = 0;
  }
}

// --------------------------------------------------------------------------- hit pass ----
// 8 warps per tile: warp w owns pixel half (w & 1) and candidates (w >> 1) + 4j of the window.
// REF: the hit decision in the reference kernels' arithmetic (frame.hit_arith = 1).
template <bool REF>
__global__ void __launch_bounds__(256, 6) k_hits(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, const int32_t* __restrict__ sorted_prims, int W, int H, int ntx,
    float thr, float bound2, const int32_t* __restrict__ active, const int32_t* __restrict__ active_count, int lo,
    int hi, const float4* __restrict__ px_state, uint32_t* __restrict__ masks32, uint32_t* __restrict__ pair_base,
    int32_t* __restrict__ prim_cnt, int32_t* __restrict__ counters, int64_t max_records,
    int32_t* __restrict__ status, int32_t* __restrict__ reset_count) {
  chain_wait();
  chain_release();
  __shared__ uint32_t s_m[2][kWinMax];
  __shared__ int32_t s_pref[kWinMax];
  __shared__ int warp_sums[32];
  __shared__ int s_tile_base;
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  // a view of a batch clears the count of the list its compositing pass of this wave will append to (the
  // per-primitive scan does that for a frame rendered alone)
  if (reset_count && blockIdx.x == 0 && threadIdx.x == 0) *reset_count = 0;
  const int n_active = *active_count;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = warp & 1;
  for (int slot_i = blockIdx.x; slot_i < n_active; slot_i += gridDim.x) {
  const int tile = active[slot_i];
  const int s = tile_offsets[tile];
  const int len = tile_len[tile];
  const int wlo = min(lo, len), whi = min(hi, len);
  const int nwin = whi - wlo;
  if (nwin <= 0) continue;
  const TilePix tp = tile_pixel(tile, half * 32 + lane, ntx, W, H);
  V3 o = {0.f, 0.f, 0.f}, d = {0.f, 0.f, 0.f};
  bool act = false;
  if (tp.valid) {
    o = load3(rays_o, tp.pix); d = load3(rays_d, tp.pix);
    act = px_state[tp.pix].w >= MLPSP_TERM;
  }
  // The 32 rays of this warp normally leave one origin; then R^T (c - o) is a per-candidate constant, computed by
  // one lane per candidate for a batch of 32 candidates and handed round by shuffles (same operations on the
  // same inputs: same bits as computing it in every lane).
  const uint32_t vmask = __ballot_sync(0xffffffffu, tp.valid);
  V3 o0 = o;
  bool uni = false;
  if (vmask) {
    const int src = __ffs(vmask) - 1;
    o0.x = __shfl_sync(0xffffffffu, o.x, src); o0.y = __shfl_sync(0xffffffffu, o.y, src); o0.z = __shfl_sync(0xffffffffu, o.z, src);
    uni = __all_sync(0xffffffffu, !tp.valid || (o.x == o0.x && o.y == o0.y && o.z == o0.z));
  }
  for (int b0 = wlo + (warp >> 1); b0 < whi; b0 += 128) {
    const int il = b0 + 4 * lane;
    int pl = -1;
    V3 vll = {0.f, 0.f, 0.f};
    if (il < whi) {
      pl = sorted_prims[s + il];
      if (!REF && uni && pl >= 0 && pl < n) vll = local_offset(load_geom(geom, pl), o0);
    }
    const int cnt = min(32, (whi - b0 + 3) >> 2);
    for (int t = 0; t < cnt; ++t) {
      const int i = b0 + 4 * t;
      const int p = __shfl_sync(0xffffffffu, pl, t);
      const V3 vl = {__shfl_sync(0xffffffffu, vll.x, t), __shfl_sync(0xffffffffu, vll.y, t), __shfl_sync(0xffffffffu, vll.z, t)};
      bool hit = false;
      if (act && p >= 0 && p < n) {
        const Geom g = load_geom(geom, p);
        if (!surely_misses(g, o, d, bound2)) {
          Hit h;
          if (REF) hit = hit_test_ref(load_geom_ref(geom, p), o, d, thr, h);
          else hit = uni ? hit_test_t<true>(g, o, d, vl, thr, h) : hit_test_t<false>(g, o, d, vl, thr, h);
        }
      }
      const uint32_t m = __ballot_sync(0xffffffffu, hit);
      if (lane == 0) s_m[half][i - wlo] = m;
    }
  }
  __syncthreads();
  int running = 0;
  for (int j0 = 0; j0 < nwin; j0 += 256) {
    const int j = j0 + tid;
    const int c = (j < nwin) ? __popc(s_m[0][j]) + __popc(s_m[1][j]) : 0;
    int total;
    const int ex = block_exclusive_scan(c, warp_sums, total);
    if (j < nwin) s_pref[j] = running + ex;
    running += total;
  }
  if (tid == 0) {
    const int base = running > 0 ? atomicAdd(counters + kCtrRecords, running) : 0;
    s_tile_base = base;
    if ((int64_t)base + running > max_records) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_RECORD_OVERFLOW);
  }
  __syncthreads();
  const int base = s_tile_base;
  for (int j = tid; j < nwin; j += 256) {
    const uint32_t m0 = s_m[0][j], m1 = s_m[1][j];
    masks32[2 * (size_t)(s + wlo + j)] = m0;
    masks32[2 * (size_t)(s + wlo + j) + 1] = m1;
    pair_base[s + wlo + j] = (uint32_t)(base + s_pref[j]);
    const int c = __popc(m0) + __popc(m1);
    if (c > 0) atomicAdd(prim_cnt + sorted_prims[s + wlo + j], c);
  }
  __syncthreads();   // shared arrays are reused by the next tile of this CTA
  }
}

// Geometric hit masks of all pairs (no transmittance state): the superset the waves draw from.
__global__ void __launch_bounds__(256) k_hit_masks_all(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom, int n,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ sorted_prims, int W, int H, int ntx,
    float thr, float bound2, uint32_t* __restrict__ masks32, int ref_arith, const int32_t* __restrict__ status) {
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tile = blockIdx.x;
  const int s = tile_offsets[tile];
  const int len = tile_offsets[tile + 1] - s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, half = warp & 1;
  const TilePix tp = tile_pixel(tile, half * 32 + lane, ntx, W, H);
  V3 o = {0.f, 0.f, 0.f}, d = {0.f, 0.f, 0.f};
  if (tp.valid) { o = load3(rays_o, tp.pix); d = load3(rays_d, tp.pix); }
  for (int i = (warp >> 1); i < len; i += 4) {
    const int p = sorted_prims[s + i];
    bool hit = false;
    if (tp.valid && p >= 0 && p < n) {
      const Geom g = load_geom(geom, p);
      if (!surely_misses(g, o, d, bound2)) {
        Hit h;
        hit = ref_arith ? hit_test_ref(load_geom_ref(geom, p), o, d, thr, h) : hit_test(g, o, d, thr, h);
      }
    }
    const uint32_t m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) masks32[2 * (size_t)(s + i) + half] = m;
  }
}

// ------------------------------------------------------- per-primitive scan + work items ----
// A primitive's records of the wave become evaluator work items: blocks of 128 rows, and -- when the evaluator has
// a kernel for small groups (split) -- a remainder of at most 32 records becomes an item on a list of its own
// instead of a 128-row block that would be three quarters empty.  (Two small items for a remainder of 33..64
// measured slower than one block.)
__device__ __forceinline__ int items_of(int cnt, int split) {
  if (!split) return (cnt + kRowsPerItem - 1) / kRowsPerItem;
  const int rem = cnt % kRowsPerItem;
  return cnt / kRowsPerItem + (rem > kRowsPerSmallItem ? 1 : 0);
}
__device__ __forceinline__ int small_items_of(int cnt, int split) {
  if (!split) return 0;
  const int rem = cnt % kRowsPerItem;
  return (rem > 0 && rem <= kRowsPerSmallItem) ? 1 : 0;
}

__global__ void k_prim_partial(const int32_t* __restrict__ prim_cnt, int n, int split, int32_t* __restrict__ blk,
                               const int32_t* __restrict__ status) {
  chain_wait();
  chain_release();
  __shared__ int warp_sums[32];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int64_t base = (int64_t)blockIdx.x * kPrimScanItems + (int64_t)threadIdx.x * 4;
  int a = 0, b = 0, m = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (base + j < n) { const int c = prim_cnt[base + j]; a += c; b += items_of(c, split); m += small_items_of(c, split); }
  int ta, tb, tm;
  block_exclusive_scan(a, warp_sums, ta);
  block_exclusive_scan(b, warp_sums, tb);
  block_exclusive_scan(m, warp_sums, tm);
  if (threadIdx.x == 0) { blk[3 * blockIdx.x] = ta; blk[3 * blockIdx.x + 1] = tb; blk[3 * blockIdx.x + 2] = tm; }
}

// Second pass: every block sums the partial totals of the blocks before it (a few hundred at most), scans
// its own 1,024 counts, writes the CSR offsets and the evaluator's work items and clears the counts the NEXT wave
// will add to (waves alternate between two count arrays, so nothing this launch reads is written by it); the last
// block also publishes the wave's totals.  blk == nullptr: there was no first pass -- the block sums the counts
// of the blocks before it itself (worth it up to a few blocks: one launch instead of two).
__global__ void k_prim_final(const int32_t* __restrict__ prim_cnt, int32_t* __restrict__ prim_cnt_next,
                             int32_t* __restrict__ prim_cursor, int n, int split,
                             const int32_t* __restrict__ blk, int32_t* __restrict__ prim_off,
                             int4* __restrict__ work, int64_t max_work, int4* __restrict__ work_small, int64_t max_work_small,
                             int32_t* __restrict__ counters, int next_list, int32_t* __restrict__ status) {
  chain_wait();
  chain_release();
  __shared__ int warp_sums[32];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) {
    // after a record overflow, leave the size the wave asked for so the caller can grow its scratch
    if (blockIdx.x == 0 && threadIdx.x == 0 && (status[MLPSP_ST_BITS] & MLPSP_ST_RECORD_OVERFLOW))
      atomicMax(status + MLPSP_ST_WAVE_RECORDS, counters[kCtrRecords]);
    return;
  }
  int pa = 0, pb = 0, pm = 0;
  if (blk) {
    for (int i = threadIdx.x; i < (int)blockIdx.x; i += blockDim.x) { pa += blk[3 * i]; pb += blk[3 * i + 1]; pm += blk[3 * i + 2]; }
  } else {
    const int4* c4 = reinterpret_cast<const int4*>(prim_cnt);     // both count arrays start 16-byte aligned
    const int before4 = (int)blockIdx.x * (kPrimScanItems / 4);
#pragma unroll 2
    for (int i = threadIdx.x; i < before4; i += blockDim.x) {
      const int4 c = c4[i];
      pa += c.x + c.y + c.z + c.w;
      pb += items_of(c.x, split) + items_of(c.y, split) + items_of(c.z, split) + items_of(c.w, split);
      pm += small_items_of(c.x, split) + small_items_of(c.y, split) + small_items_of(c.z, split) + small_items_of(c.w, split);
    }
  }
  int base_a, base_b, base_m;
  block_exclusive_scan(pa, warp_sums, base_a);
  block_exclusive_scan(pb, warp_sums, base_b);
  block_exclusive_scan(pm, warp_sums, base_m);
  const int64_t base = (int64_t)blockIdx.x * kPrimScanItems + (int64_t)threadIdx.x * 4;
  int c[4], a = 0, b = 0, m = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    c[j] = (base + j < n) ? prim_cnt[base + j] : 0;
    a += c[j]; b += items_of(c[j], split); m += small_items_of(c[j], split);
  }
  int ta, tb, tm;
  int ea = block_exclusive_scan(a, warp_sums, ta) + base_a;
  int eb = block_exclusive_scan(b, warp_sums, tb) + base_b;
  int em = block_exclusive_scan(m, warp_sums, tm) + base_m;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (base + j < n) {
      prim_off[base + j] = ea;
      const int it = items_of(c[j], split), sm = small_items_of(c[j], split);
      for (int q = 0; q < it; ++q)
        if ((int64_t)eb + q < max_work)
          work[eb + q] = make_int4((int)(base + j), ea + q * kRowsPerItem, min(kRowsPerItem, c[j] - q * kRowsPerItem), 0);
      const int first_small = c[j] - c[j] % kRowsPerItem;     // the remainder starts behind the full blocks
      for (int q = 0; q < sm; ++q)
        if ((int64_t)em + q < max_work_small)
          work_small[em + q] = make_int4((int)(base + j), ea + first_small + q * kRowsPerSmallItem,
                                         min(kRowsPerSmallItem, c[j] - first_small - q * kRowsPerSmallItem), 0);
      ea += c[j]; eb += it; em += sm;
      prim_cnt_next[base + j] = 0;
      prim_cursor[base + j] = 0;
    }
  }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
    const int R = base_a + ta;
    int G = base_b + tb, Gs = base_m + tm;
    if ((int64_t)G > max_work) { G = (int)max_work; atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_RECORD_OVERFLOW); }
    if ((int64_t)Gs > max_work_small) { Gs = (int)max_work_small; atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_RECORD_OVERFLOW); }
    prim_off[n] = R;
    counters[kCtrWork] = G;
    counters[kCtrWorkSmall] = Gs;
    counters[kCtrWorkNext] = 0;
    counters[kCtrActive0 + next_list] = 0;   // kCtrRecords keeps counting: compositing slots are unique per frame
    if (R > 0) {
      atomicAdd((unsigned long long*)(status + MLPSP_ST_RECORDS_LO), (unsigned long long)R);
      atomicMax(status + MLPSP_ST_WAVE_RECORDS, R);
      atomicMax(status + MLPSP_ST_WORK_ITEMS, G + Gs);
      atomicAdd(status + MLPSP_ST_WORK_TOTAL, G + Gs);
      atomicAdd(status + MLPSP_ST_WORK_SMALL, Gs);
      atomicAdd(status + MLPSP_ST_WAVES, 1);
    }
  }
}

// Up to 8,192 primitives the scan is one launch.  Beyond that the block that sums the most counts becomes the
// launch's critical path (100,000 primitives: 23 us in one launch against 18 us in two).
constexpr int kPrimScanSoloBlocks = 8;

int launch_prim_scan(const Scratch& s, int n, int next_list, int32_t* status, cudaStream_t st, bool split_small, int wave) {
  const int nblk = (n + kPrimScanItems - 1) / kPrimScanItems;
  if (nblk == 0) return MLPSP_OK;
  const bool solo = nblk <= kPrimScanSoloBlocks;
  LaunchScope scope(kKScan, solo ? 1 : 2, st);
  const int split = split_small && s.work_small ? 1 : 0;
  const int32_t* cnt = s.prim_cnt + (size_t)(wave & 1) * prim_cnt_stride(n);
  int32_t* cnt_next = s.prim_cnt + (size_t)((wave & 1) ^ 1) * prim_cnt_stride(n);
  if (!solo) launch_chained(k_prim_partial, dim3(nblk), dim3(kPrimScanItems / 4), 0, st, cnt, n, split, s.scan_blk, status);
  launch_chained(k_prim_final, dim3(nblk), dim3(kPrimScanItems / 4), 0, st, cnt, cnt_next, s.prim_cursor, n, split, solo ? nullptr : s.scan_blk, s.prim_off, s.work,
                                     s.max_work, s.work_small, s.max_work_small, s.counters, next_list, status);
  return cuda_check(cudaGetLastError(), "prim_scan");
}

// -------------------------------------------------------------------------- fill pass ----
// Feature gates (semantic_tetra_gates, np_tile_kernels.cu:97-124).
__device__ __forceinline__ float4 tetra_gates(const Hit& h, float lsx, float lsy, float lsz, float beta, float tau) {
  const float sx = det_exp(lsx), sy = det_exp(lsy), sz = det_exp(lsz);
  const float ux = fminf(1.f, fmaxf(-1.f, h.qx / (beta * sx + 1e-6f)));
  const float uy = fminf(1.f, fmaxf(-1.f, h.qy / (beta * sy + 1e-6f)));
  const float uz = fminf(1.f, fmaxf(-1.f, h.qz / (beta * sz + 1e-6f)));
  const float l0 = tau * (ux + uy + uz), l1 = tau * (ux - uy - uz);
  const float l2 = tau * (-ux + uy - uz), l3 = tau * (-ux - uy + uz);
  const float lm = fmaxf(fmaxf(l0, l1), fmaxf(l2, l3));
  const float e0 = __expf(l0 - lm), e1 = __expf(l1 - lm), e2 = __expf(l2 - lm), e3 = __expf(l3 - lm);
  const float inv = 1.f / fmaxf(e0 + e1 + e2 + e3, 1e-8f);
  return make_float4(e0 * inv, e1 * inv, e2 * inv, e3 * inv);
}

// One CTA per active tile.  Pairs with hits reserve their primitive-major range (one atomic per pair),
// then threads walk the tile's RECORDS (not its pixels): record r of the tile-wave belongs to the pair
// found by binary search in the slot prefix, and to the pixel of the (r - prefix)-th set mask bit.
__global__ void __launch_bounds__(256) k_fill(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, const int32_t* __restrict__ sorted_prims, int W, int H, int ntx,
    float thr, const int32_t* __restrict__ active, const int32_t* __restrict__ active_count, int lo, int hi,
    const uint32_t* __restrict__ masks32, const uint32_t* __restrict__ pair_base,
    const int32_t* __restrict__ prim_off, int32_t* __restrict__ prim_cursor, RecIn* __restrict__ rec_in,
    float* __restrict__ rec_t, float4* __restrict__ rec_gate, float beta, float tau, int exact_hits, int ref_arith,
    const int32_t* __restrict__ status) {
  chain_wait();
  chain_release();
  __shared__ uint32_t s_m[2][kWinMax];
  __shared__ int32_t s_pref[kWinMax + 1];   // slot of the pair's first record, relative to the tile-wave
  __shared__ int32_t s_q0[kWinMax];         // primitive-major position of the pair's first record
  __shared__ float s_ray[64][6];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int n_active = *active_count;
  const int tid = threadIdx.x;
  for (int slot_i = blockIdx.x; slot_i < n_active; slot_i += gridDim.x) {
  const int tile = active[slot_i];
  const int s = tile_offsets[tile];
  const int len = tile_len[tile];
  const int wlo = min(lo, len), whi = min(hi, len);
  const int nwin = whi - wlo;
  if (nwin <= 0) continue;
  if (tid < 64) {
    const TilePix tp = tile_pixel(tile, tid, ntx, W, H);
    V3 o = {0.f, 0.f, 0.f}, d = {0.f, 0.f, 0.f};
    if (tp.valid) { o = load3(rays_o, tp.pix); d = load3(rays_d, tp.pix); }
    s_ray[tid][0] = o.x; s_ray[tid][1] = o.y; s_ray[tid][2] = o.z;
    s_ray[tid][3] = d.x; s_ray[tid][4] = d.y; s_ray[tid][5] = d.z;
  }
  const uint32_t slot_base = pair_base[s + wlo];
  for (int j = tid; j < nwin; j += 256) {
    const uint32_t m0 = masks32[2 * (size_t)(s + wlo + j)], m1 = masks32[2 * (size_t)(s + wlo + j) + 1];
    s_m[0][j] = m0; s_m[1][j] = m1;
    s_pref[j] = (int32_t)(pair_base[s + wlo + j] - slot_base);
    const int c = __popc(m0) + __popc(m1);
    int q0 = 0;
    if (c > 0) {
      const int p = sorted_prims[s + wlo + j];
      q0 = prim_off[p] + atomicAdd(prim_cursor + p, c);
    }
    s_q0[j] = q0;
    if (j == nwin - 1) s_pref[nwin] = s_pref[j] + c;
  }
  __syncthreads();
  const int total = s_pref[nwin];
  for (int r = tid; r < total; r += 256) {
    int a = 0, b = nwin - 1;                 // largest j with s_pref[j] <= r (empty pairs share a prefix
    while (a < b) {                          //  with their successor, so the last such j is the owner)
      const int mid = (a + b + 1) >> 1;
      if (s_pref[mid] <= r) a = mid; else b = mid - 1;
    }
    const int j = a, k = r - s_pref[a];
    const uint32_t m0 = s_m[0][j], m1 = s_m[1][j];
    const int c0 = __popc(m0);
    const int px = (k < c0) ? nth_set_bit(m0, k) : 32 + nth_set_bit(m1, k - c0);
    const int p = sorted_prims[s + wlo + j];
    const V3 o = {s_ray[px][0], s_ray[px][1], s_ray[px][2]}, d = {s_ray[px][3], s_ray[px][4], s_ray[px][5]};
    Hit ht;
    // the pair is known to hit: values only.  The feature gates divide the local offset by the scales, which
    // magnifies its rounding, so frames with features keep the decision-grade arithmetic.
    // Per-pixel ordering sorts by t: its order must be the decision-grade one too.
    if (ref_arith) hit_test_ref(load_geom_ref(geom, p), o, d, thr, ht);    // the reference kernels' own values
    else if (rec_gate || exact_hits) hit_test(load_geom(geom, p), o, d, thr, ht);
    else hit_values_fast(load_geom(geom, p), o, d, ht);
    const uint32_t slot = slot_base + (uint32_t)r;
    RecIn rec;
    rec.rdx = d.x; rec.rdy = d.y; rec.rdz = d.z; rec.dx = ht.dx; rec.dy = ht.dy; rec.dz = ht.dz;
    rec.decay = ht.decay; rec.slot = slot;
    rec_in[s_q0[j] + k] = rec;
    if (rec_t) rec_t[slot] = ht.t;
    if (rec_gate) {
      const float4 ls = __ldg(geom + (size_t)p * 4 + 3);
      rec_gate[slot] = tetra_gates(ht, ls.x, ls.y, ls.z, beta, tau);
    }
  }
  __syncthreads();   // shared arrays are reused by the next tile of this CTA
  }
}

// --------------------------------------------------------------------------- composite ----
// 64 threads per tile; each warp owns 32 pixels and stops as soon as none of them is live.
struct PrimStats {
  const float* gt_rgb; const int32_t* sorted_prims;
  float* sum_w; float* max_w; int32_t* hits; float* sum_werr; int32_t* contrib;
};

template <bool STATS>
__global__ void __launch_bounds__(64) k_composite(
    PrimStats ps,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, int W, int H, int ntx, const int32_t* __restrict__ active,
    const int32_t* __restrict__ active_count, int lo, int hi, const uint32_t* __restrict__ masks32,
    const uint32_t* __restrict__ pair_base, const float4* __restrict__ rec_out, const float* __restrict__ rec_t,
    float4* __restrict__ px_state, float2* __restrict__ px_depth, float* __restrict__ rgb,
    float* __restrict__ alpha, float* __restrict__ depth_t, uint32_t* __restrict__ mask_used32,
    float* __restrict__ rec_w, float* __restrict__ rec_tr, float bgr, float bgg, float bgb, int has_bg,
    int32_t* __restrict__ next_active,
    int32_t* __restrict__ next_count, int32_t* __restrict__ status) {
  chain_wait();
  chain_release();
  __shared__ int s_live[2];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int n_active = *active_count;
  for (int slot_i = blockIdx.x; slot_i < n_active; slot_i += gridDim.x) {
  const int tile = active[slot_i];
  const int s = tile_offsets[tile];
  const int len = tile_len[tile];
  const int wlo = min(lo, len), whi = min(hi, len);
  const int lane = threadIdx.x & 31, half = threadIdx.x >> 5;
  const TilePix tp = tile_pixel(tile, half * 32 + lane, ntx, W, H);
  float4 st = make_float4(0.f, 0.f, 0.f, 0.f);
  float2 dp = make_float2(0.f, 0.f);
  if (tp.valid) { st = px_state[tp.pix]; if (depth_t) dp = px_depth[tp.pix]; }
  bool act = tp.valid && st.w >= MLPSP_TERM;
  const uint32_t lt = (1u << lane) - 1u;
  int used = 0;
  float gtr = 0.f, gtg = 0.f, gtb = 0.f;
  if (STATS && tp.valid) { gtr = ps.gt_rgb[(size_t)tp.pix * 3]; gtg = ps.gt_rgb[(size_t)tp.pix * 3 + 1]; gtb = ps.gt_rgb[(size_t)tp.pix * 3 + 2]; }
  for (int i0 = wlo; i0 < whi && __any_sync(0xffffffffu, act); i0 += 32) {
    const int idx = i0 + lane;
    uint2 mm = make_uint2(0u, 0u);
    uint32_t bb = 0;
    if (idx < whi) {
      mm = *reinterpret_cast<const uint2*>(masks32 + 2 * (size_t)(s + idx));
      bb = pair_base[s + idx];
    }
    const int cnt = min(32, whi - i0);
    bool stop = false;
    // four pairs at a time: the records a lane may need are requested first (whether its pixel is still live or
    // not), then blended in list order, so the gathers of a batch overlap instead of forming a chain
    for (int j0 = 0; j0 < cnt && !stop; j0 += 4) {
      float4 rr[4];
      uint32_t slot4[4], m04[4], mine4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = min(j0 + u, 31);
        const uint32_t m0 = __shfl_sync(0xffffffffu, mm.x, j), m1 = __shfl_sync(0xffffffffu, mm.y, j);
        const uint32_t b = __shfl_sync(0xffffffffu, bb, j);
        const uint32_t mine = (j0 + u < cnt) ? (half ? m1 : m0) : 0u;
        m04[u] = m0; mine4[u] = mine;
        slot4[u] = b + (half ? __popc(m0) : 0) + __popc(mine & lt);
        rr[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((mine >> lane) & 1u) rr[u] = rec_out[slot4[u]];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u;
        const uint32_t mine = mine4[u];
        if (stop || mine == 0u) continue;
        const bool take = act && ((mine >> lane) & 1u);
        float sw = 0.f, swerr = 0.f;
        if (take) {
          const uint32_t slot = slot4[u];
          const float4 r = rr[u];
          const float w = st.w * r.w;
          st.x = fmaf(w, r.x, st.x); st.y = fmaf(w, r.y, st.y); st.z = fmaf(w, r.z, st.z);
          if (STATS) {
            sw = w;
            if (w > 1e-1f) swerr = w * (fabsf(st.x - gtr) + fabsf(st.y - gtg) + fabsf(st.z - gtb));
          }
          if (depth_t) { dp.x = fmaf(w, rec_t[slot], dp.x); dp.y += w; }
          if (rec_w) rec_w[slot] = w;
          if (rec_tr) rec_tr[slot] = st.w;
          st.w *= (1.f - r.w);
          act = st.w >= MLPSP_TERM;
        }
        const uint32_t um = __ballot_sync(0xffffffffu, take);
        if (STATS && um) {
          // this half-tile's share of the pair's statistics: one atomic per array
          const int n_hit = __popc(__ballot_sync(0xffffffffu, sw > 1e-8f));
          const int n_con = __popc(__ballot_sync(0xffffffffu, sw > 1e-1f));
          float tsum = sw, tmax = sw, terr = swerr;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
            terr += __shfl_xor_sync(0xffffffffu, terr, o);
          }
          if (lane == 0) {
            const int p = ps.sorted_prims[s + i0 + j];
            atomicAdd(ps.sum_w + p, tsum);
            atomicMax(reinterpret_cast<int*>(ps.max_w + p), __float_as_int(tmax));   // w >= 0: bit order = value order
            if (n_hit) atomicAdd(ps.hits + p, n_hit);
            if (n_con) { atomicAdd(ps.contrib + p, n_con); atomicAdd(ps.sum_werr + p, terr); }
          }
        }
        if (um) {
          if (lane == 0) { used += __popc(um); if (mask_used32) mask_used32[2 * (size_t)(s + i0 + j) + half] = um; }
          if (!__any_sync(0xffffffffu, act)) stop = true;
        }
        (void)m04;
      }
    }
  }
  if (tp.valid) {
    px_state[tp.pix] = st;
    const float a = 1.f - st.w;
    float r = st.x, g = st.y, b = st.z;
    if (has_bg) {
      const float k = fminf(fmaxf(1.f - a, 0.f), 1.f);
      r += k * bgr; g += k * bgg; b += k * bgb;
    }
    rgb[(size_t)tp.pix * 3] = r; rgb[(size_t)tp.pix * 3 + 1] = g; rgb[(size_t)tp.pix * 3 + 2] = b;
    alpha[tp.pix] = a;
    if (depth_t) { px_depth[tp.pix] = dp; depth_t[tp.pix] = dp.x / ((dp.y > 1e-8f) ? dp.y : 1.f); }
  }
  const bool live = __any_sync(0xffffffffu, act);
  if (lane == 0) {
    s_live[half] = live;
    if (used) atomicAdd((unsigned long long*)(status + MLPSP_ST_USED_LO), (unsigned long long)used);
  }
  __syncthreads();
  if (threadIdx.x == 0 && (s_live[0] | s_live[1]) && whi < len) next_active[atomicAdd(next_count, 1)] = tile;
  __syncthreads();
  }
}

// --------------------------------------------------------------- per-pixel exact ordering ----
// render_tiles_kernel_with_sort (np_tile_kernels.cu:714-926): every pixel sorts its own hits by its own hit
// distance and blends them front to back.  Here the hits of all pixels have been found and evaluated in one
// wave (no pixel is gated by transmittance, as the order is not known yet); a thread per pixel collects its
// (t, record slot) pairs in list order -- at most kPixelHits, one more raises MLPSP_ST_PIXEL_HITS and the pixel
// blends what it has, as the reference's kernel does before its wrapper raises -- sorts them with the
// reference's stable insertion sort (ties keep list order) and blends until the transmittance falls below 1e-3.
// With a feature map (render_tiles_kernel_with_sort_and_feat) the consumed records and their weights are left for
// k_feature_composite, whose sum does not depend on the order.
constexpr int kPixelHits = 256;
__global__ void __launch_bounds__(64) k_composite_per_pixel(
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, int T, int W, int H, int ntx,
    const uint32_t* __restrict__ masks32, const uint32_t* __restrict__ pair_base, const float4* __restrict__ rec_out,
    const float* __restrict__ rec_t, float* __restrict__ rgb, float* __restrict__ alpha, float bgr, float bgg, float bgb,
    int has_bg, uint32_t* __restrict__ used32, float* __restrict__ rec_w, int32_t* __restrict__ status) {
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int lane = threadIdx.x & 31, half = threadIdx.x >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  for (int tile = blockIdx.x; tile < T; tile += gridDim.x) {
    const int s = tile_offsets[tile], len = tile_len[tile];
    const TilePix tp = tile_pixel(tile, half * 32 + lane, ntx, W, H);
    float key[kPixelHits];
    uint32_t slot[kPixelHits];
    uint16_t pair[kPixelHits];               // position in the tile's list (< 2048), for the consumed masks
    int cnt = 0;
    bool over = false;
    int used = 0;
    for (int i = 0; i < len && !over; ++i) {
      const uint32_t m0 = masks32[2 * (size_t)(s + i)], m1 = masks32[2 * (size_t)(s + i) + 1];
      const uint32_t mine = half ? m1 : m0;
      if (tp.valid && ((mine >> lane) & 1u)) {
        if (cnt < kPixelHits) {
          const uint32_t sl = pair_base[s + i] + (half ? __popc(m0) : 0) + __popc(mine & lt);
          key[cnt] = rec_t[sl];
          slot[cnt] = sl;
          pair[cnt] = (uint16_t)i;
          ++cnt;
        } else {
          over = true;
        }
      }
    }
    if (over) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_PIXEL_HITS);
    for (int i = 1; i < cnt; ++i) {
      const float kt = key[i];
      const uint32_t ks = slot[i];
      const uint16_t kp = pair[i];
      int j = i - 1;
      while (j >= 0 && key[j] > kt) { key[j + 1] = key[j]; slot[j + 1] = slot[j]; pair[j + 1] = pair[j]; --j; }
      key[j + 1] = kt;
      slot[j + 1] = ks;
      pair[j + 1] = kp;
    }
    float cr = 0.f, cg = 0.f, cb = 0.f, trans = 1.f;
    for (int i = 0; i < cnt; ++i) {
      const float4 r = rec_out[slot[i]];
      const float w = trans * r.w;
      cr = fmaf(w, r.x, cr); cg = fmaf(w, r.y, cg); cb = fmaf(w, r.z, cb);
      if (rec_w) {
        // the feature pass adds w * (gated attributes) for every consumed record, whatever their order
        rec_w[slot[i]] = w;
        atomicOr(used32 + 2 * (size_t)(s + pair[i]) + half, 1u << lane);
      }
      trans *= (1.f - r.w);
      ++used;
      if (trans < MLPSP_TERM) break;
    }
    if (tp.valid) {
      const float a = 1.f - trans;
      if (has_bg) {
        const float k = fminf(fmaxf(1.f - a, 0.f), 1.f);
        cr += k * bgr; cg += k * bgg; cb += k * bgb;
      }
      rgb[(size_t)tp.pix * 3] = cr; rgb[(size_t)tp.pix * 3 + 1] = cg; rgb[(size_t)tp.pix * 3 + 2] = cb;
      alpha[tp.pix] = a;
    }
    for (int o = 16; o > 0; o >>= 1) used += __shfl_xor_sync(0xffffffffu, used, o);
    if (lane == 0 && used) atomicAdd((unsigned long long*)(status + MLPSP_ST_USED_LO), (unsigned long long)used);
  }
}

// ------------------------------------------------------------------- feature compositing ----
// out_feat[pix, :] = sum over the pixel's composited records of w * mix(p, gates)  with
//   S = 4: mix = sum_s g_s * attr[p, s, :]      S = 5: mix = attr[p, 0, :] + sum_s g_s * attr[p, 1+s, :]
//   S = 1: mix = attr[p, 0, :]                                     (np_tile_kernels.cu:6036-6075)
// One CTA per tile after the last wave.  The 64 x C accumulator tile lives in shared memory; for
// every pair that composited at least one record, the consumed pixels and their coefficients
// w * g_s are compacted into shared memory and every thread adds its channels' contribution.
constexpr int kFeatThreads = 256;
constexpr int kFeatBatch = 256;    // consumed records staged per barrier (one per thread)
constexpr int kFeatChan = 256;     // channels per CTA: (tile, channel block) pairs make the grid

// Shared memory: [64][CB] accumulators, then the tile's consumed masks and their record prefix.
template <bool VEC4>
__global__ void __launch_bounds__(kFeatThreads) k_feature_composite(
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, const int32_t* __restrict__ sorted_prims, int W, int H, int ntx,
    const uint32_t* __restrict__ used32, const uint32_t* __restrict__ masks32, const uint32_t* __restrict__ pair_base,
    const float* __restrict__ rec_w, const float4* __restrict__ rec_gate, const float* __restrict__ feat_attr,
    int S, int C, int CB, float* __restrict__ out_feat, const int32_t* __restrict__ status) {
  extern __shared__ float s_acc[];                 // [64][CB]
  __shared__ uint32_t s_u[2][kWinMax];             // consumed masks of the tile's pairs
  __shared__ int32_t s_pref[kWinMax + 1];          // records before pair i
  __shared__ __align__(16) float s_cw[kFeatBatch][8];   // per staged record: base weight + 4 gated weights (+ padding)
  __shared__ int s_px[kFeatBatch];                 // its pixel
  __shared__ int s_pr[kFeatBatch];                 // its primitive
  __shared__ int s_run[kFeatBatch + 1];            // first staged record of every run of equal primitives
  __shared__ int s_nruns;
  __shared__ int warp_sums[32];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tile = blockIdx.x, c0 = blockIdx.y * CB;
  const int nc = min(CB, C - c0);
  // VEC4 (launched for maps of at least 256 channels, a multiple of 4): full 256-channel blocks take the
  // four-channels-per-thread path; narrower blocks measured no faster with it and keep the leaner kernel
  const bool vec4 = VEC4 && nc == kFeatChan;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < 64 * CB; i += kFeatThreads) s_acc[i] = 0.f;
  const int s = tile_offsets[tile];
  const int len = min(tile_len[tile], kWinMax);
  int running = 0;
  for (int j0 = 0; j0 < len; j0 += kFeatThreads) {
    const int j = j0 + tid;
    uint32_t u0 = 0u, u1 = 0u;
    if (j < len) { u0 = used32[2 * (size_t)(s + j)]; u1 = used32[2 * (size_t)(s + j) + 1]; s_u[0][j] = u0; s_u[1][j] = u1; }
    int total;
    const int ex = block_exclusive_scan(__popc(u0) + __popc(u1), warp_sums, total);
    if (j < len) s_pref[j] = running + ex;
    running += total;
  }
  if (tid == 0) s_pref[len] = running;
  __syncthreads();
  const int n_tot = running;
  for (int b0 = 0; b0 < n_tot; b0 += kFeatBatch) {
    const int n = min(kFeatBatch, n_tot - b0);
    if (tid < n) {
      const int r = b0 + tid;
      int a = 0, b = len - 1;                  // largest pair index with s_pref <= r (see k_fill)
      while (a < b) {
        const int mid = (a + b + 1) >> 1;
        if (s_pref[mid] <= r) a = mid; else b = mid - 1;
      }
      const int k = r - s_pref[a];
      const uint32_t u0 = s_u[0][a], u1 = s_u[1][a];
      const int cu0 = __popc(u0);
      const int px = (k < cu0) ? nth_set_bit(u0, k) : 32 + nth_set_bit(u1, k - cu0);
      const uint32_t m0 = masks32[2 * (size_t)(s + a)], m1 = masks32[2 * (size_t)(s + a) + 1];
      const uint32_t slot = pair_base[s + a] +
                            (px < 32 ? __popc(m0 & ((1u << px) - 1u)) : __popc(m0) + __popc(m1 & ((1u << (px - 32)) - 1u)));
      const float w = rec_w[slot];
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
      if (S > 1) g = rec_gate[slot];
      s_px[tid] = px;
      const int prim = sorted_prims[s + a];
      s_pr[tid] = prim;
      s_cw[tid][0] = w; s_cw[tid][1] = w * g.x; s_cw[tid][2] = w * g.y; s_cw[tid][3] = w * g.z; s_cw[tid][4] = w * g.w;
      // the first record of a pair asks L2 for the pair's attribute rows of this channel block
      if (k == 0 || tid == 0) {
        const char* rows = reinterpret_cast<const char*>(feat_attr + (size_t)prim * S * C + c0);
        for (int sl = 0; sl < S; ++sl)
          for (int b = 0; b < nc * 4; b += 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(rows + (size_t)sl * C * 4 + b));
      }
    }
    __syncthreads();
    // runs of equal primitives (block-wide compaction of the run heads)
    {
      const bool head = tid < n && (tid == 0 || s_pr[tid] != s_pr[tid - 1]);
      int total;
      const int pos = block_exclusive_scan(head ? 1 : 0, warp_sums, total);
      if (head) s_run[pos] = tid;
      if (tid == 0) { s_run[total] = n; s_nruns = total; }
    }
    __syncthreads();
    const int nruns = s_nruns;
    // A thread owns one channel; with fewer than 256 channels in the block, RL threads of a warp share a channel
    // and split the records of a run between them (one primitive touches a pixel at most once, so the records
    // of a run hit distinct accumulator cells; runs follow one another in warp lockstep).  The attribute rows
    // of run r + 2 are requested before run r is accumulated, so their latency overlaps two runs of arithmetic.
    if (vec4) {
      // four adjacent channels per thread: one 16-byte accumulator update serves four channels, and the record
      // coefficients are read once for them (same operations per channel as below, so the same bits)
      const int ng = nc >> 2;
      int RL = 1;
      while (RL < 32 && 2 * RL * ng <= kFeatThreads) RL *= 2;
      const int CPW = 32 / RL, rl = lane / CPW;
      uint32_t wmask = 0xffffffffu;
      for (int g = warp * CPW + lane % CPW;; g += (kFeatThreads / 32) * CPW) {
        wmask = __ballot_sync(wmask, g < ng);
        if (g >= ng) break;
        const int c = g * 4;
        const int C4 = C >> 2;
        auto load_rows = [&](int r, float4 (&a)[5]) {
          a[0] = a[1] = a[2] = a[3] = a[4] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (r >= nruns) return;
          const float4* src = reinterpret_cast<const float4*>(feat_attr + (size_t)s_pr[s_run[r]] * S * C + c0 + c);
          a[0] = __ldg(src);
          if (S >= 4) { a[1] = __ldg(src + C4); a[2] = __ldg(src + 2 * C4); a[3] = __ldg(src + 3 * C4); }
          if (S == 5) a[4] = __ldg(src + 4 * C4);
        };
        float4 a_cur[5], a_n1[5], a_n2[5];
        load_rows(0, a_cur);
        load_rows(1, a_n1);
        for (int r = 0; r < nruns; ++r) {
          load_rows(r + 2, a_n2);
          const int j0 = s_run[r], j1 = s_run[r + 1];
          auto mix = [&](const float (&cw)[5], float a0, float a1, float a2, float a3, float a4) {
            float v;
            if (S == 4) {
              v = cw[1] * a0;
              v = fmaf(cw[2], a1, v); v = fmaf(cw[3], a2, v); v = fmaf(cw[4], a3, v);
            } else if (S == 5) {
              v = cw[0] * a0;
              v = fmaf(cw[1], a1, v); v = fmaf(cw[2], a2, v); v = fmaf(cw[3], a3, v); v = fmaf(cw[4], a4, v);
            } else {
              v = cw[0] * a0;
            }
            return v;
          };
          auto contribution = [&](int j) {
            const float4 c03 = *reinterpret_cast<const float4*>(&s_cw[j][0]);
            const float cw[5] = {c03.x, c03.y, c03.z, c03.w, s_cw[j][4]};
            return make_float4(mix(cw, a_cur[0].x, a_cur[1].x, a_cur[2].x, a_cur[3].x, a_cur[4].x),
                               mix(cw, a_cur[0].y, a_cur[1].y, a_cur[2].y, a_cur[3].y, a_cur[4].y),
                               mix(cw, a_cur[0].z, a_cur[1].z, a_cur[2].z, a_cur[3].z, a_cur[4].z),
                               mix(cw, a_cur[0].w, a_cur[1].w, a_cur[2].w, a_cur[3].w, a_cur[4].w));
          };
          int j = j0 + rl;
          for (; j + RL < j1; j += 2 * RL) {
            float4* q0 = reinterpret_cast<float4*>(s_acc + s_px[j] * CB + c);
            float4* q1 = reinterpret_cast<float4*>(s_acc + s_px[j + RL] * CB + c);
            const float4 v0 = contribution(j), v1 = contribution(j + RL);
            const float4 x0 = *q0, x1 = *q1;
            *q0 = make_float4(x0.x + v0.x, x0.y + v0.y, x0.z + v0.z, x0.w + v0.w);
            *q1 = make_float4(x1.x + v1.x, x1.y + v1.y, x1.z + v1.z, x1.w + v1.w);
          }
          for (; j < j1; j += RL) {
            float4* q0 = reinterpret_cast<float4*>(s_acc + s_px[j] * CB + c);
            const float4 v0 = contribution(j), x0 = *q0;
            *q0 = make_float4(x0.x + v0.x, x0.y + v0.y, x0.z + v0.z, x0.w + v0.w);
          }
          if (RL > 1) __syncwarp(wmask);
#pragma unroll
          for (int q = 0; q < 5; ++q) { a_cur[q] = a_n1[q]; a_n1[q] = a_n2[q]; }
        }
      }
      __syncthreads();
      continue;
    }
    int RL = 1;
    while (RL < 32 && 2 * RL * nc <= kFeatThreads) RL *= 2;
    const int CPW = 32 / RL, rl = lane / CPW;
    uint32_t wmask = 0xffffffffu;              // lanes of this warp that still own a channel
    for (int c = warp * CPW + lane % CPW;; c += (kFeatThreads / 32) * CPW) {
      wmask = __ballot_sync(wmask, c < nc);
      if (c >= nc) break;
      auto load_rows = [&](int r, float (&a)[5]) {
        a[0] = a[1] = a[2] = a[3] = a[4] = 0.f;
        if (r >= nruns) return;
        const float* src = feat_attr + (size_t)s_pr[s_run[r]] * S * C + c0 + c;
        a[0] = __ldg(src);
        if (S >= 4) { a[1] = __ldg(src + C); a[2] = __ldg(src + 2 * C); a[3] = __ldg(src + 3 * C); }
        if (S == 5) a[4] = __ldg(src + 4 * C);
      };
      float a_cur[5], a_n1[5], a_n2[5];
      load_rows(0, a_cur);
      load_rows(1, a_n1);
      for (int r = 0; r < nruns; ++r) {
        load_rows(r + 2, a_n2);
        const int j0 = s_run[r], j1 = s_run[r + 1];
        auto contribution = [&](int j) {
          float v;
          if (S == 4) {
            v = s_cw[j][1] * a_cur[0];
            v = fmaf(s_cw[j][2], a_cur[1], v); v = fmaf(s_cw[j][3], a_cur[2], v); v = fmaf(s_cw[j][4], a_cur[3], v);
          } else if (S == 5) {
            v = s_cw[j][0] * a_cur[0];
            v = fmaf(s_cw[j][1], a_cur[1], v); v = fmaf(s_cw[j][2], a_cur[2], v);
            v = fmaf(s_cw[j][3], a_cur[3], v); v = fmaf(s_cw[j][4], a_cur[4], v);
          } else {
            v = s_cw[j][0] * a_cur[0];
          }
          return v;
        };
        int j = j0 + rl;
        // records of one pair touch distinct pixels: four accumulator cells are loaded together
        for (; j + 3 * RL < j1; j += 4 * RL) {
          float* q0 = s_acc + s_px[j] * CB + c; float* q1 = s_acc + s_px[j + RL] * CB + c;
          float* q2 = s_acc + s_px[j + 2 * RL] * CB + c; float* q3 = s_acc + s_px[j + 3 * RL] * CB + c;
          const float v0 = contribution(j), v1 = contribution(j + RL), v2 = contribution(j + 2 * RL), v3 = contribution(j + 3 * RL);
          const float x0 = *q0, x1 = *q1, x2 = *q2, x3 = *q3;
          *q0 = x0 + v0; *q1 = x1 + v1; *q2 = x2 + v2; *q3 = x3 + v3;
        }
        for (; j < j1; j += RL) s_acc[s_px[j] * CB + c] += contribution(j);
        if (RL > 1) __syncwarp(wmask);
#pragma unroll
        for (int q = 0; q < 5; ++q) { a_cur[q] = a_n1[q]; a_n1[q] = a_n2[q]; }
      }
    }
    __syncthreads();
  }
  for (int k = warp; k < 64; k += kFeatThreads / 32) {
    const TilePix tp = tile_pixel(tile, k, ntx, W, H);
    if (!tp.valid) continue;
    for (int c = lane; c < nc; c += 32) out_feat[(size_t)tp.pix * C + c0 + c] = s_acc[k * CB + c];
  }
}

// ------------------------------------------------------------------------------ driver ----
// after the tile pre-test a tile's list rarely holds more than a few hundred candidates, and few tiles
// need more than the first hundred: the tail wave takes whatever is left
static const int kDefaultWaves[] = {32, 32, 64, 128, 256, INT_MAX};

int launch_hit_masks(const mlpsp_scene* sc, const mlpsp_frame* fr, uint64_t* mask_geo, cudaStream_t st) {
  const int T = num_tiles(fr->width, fr->height, fr->tile);
  const int ntx = (fr->width + 7) / 8;
  LaunchScope scope(kKHits, 1, st);
  k_hit_masks_all<<<T, 256, 0, st>>>(fr->rays_o, fr->rays_d, (const float4*)sc->geom, sc->n, fr->tile_offsets,
                                     fr->sorted_prims, fr->width, fr->height, ntx, fr->threshold,
                                     miss_bound2(fr->threshold), (uint32_t*)mask_geo, fr->hit_arith == 1 ? 1 : 0, fr->status);
  return cuda_check(cudaGetLastError(), "hit_masks");
}

int launch_render_sorted(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st,
                         bool lists_refined) {
  const int W = fr->width, H = fr->height;
  const int T = num_tiles(W, H, 8);
  const int ntx = (W + 7) / 8;
  const int64_t P = (int64_t)W * H;
  const int n = sc->n;
  float bg[3] = {0.f, 0.f, 0.f};
  const int has_bg = fr->bg_color != nullptr;
  if (has_bg) { bg[0] = fr->bg_color[0]; bg[1] = fr->bg_color[1]; bg[2] = fr->bg_color[2]; }
  const bool want_t = fr->depth_t != nullptr;
  const bool want_feat = fr->feat != nullptr;
  if (want_feat) {
    MLPSP_REQUIRE(sc->feat_attr && sc->feat_dim > 0 && sc->feat_dim <= 512, MLPSP_E_ARG,
                  "feature rendering needs feat_attr with 1..512 channels");
    MLPSP_REQUIRE(sc->feat_slots == 1 || sc->feat_slots == 4 || sc->feat_slots == 5, MLPSP_E_ARG,
                  "feature slots must be 1, 4 or 5");
  }
  const bool keep = fr->keep_records == 1;
  const bool want_stats = fr->stat_sum_w != nullptr;
  const bool per_pixel = fr->sort_key == MLPSP_ORDER_PER_PIXEL;
  if (per_pixel) {
    MLPSP_REQUIRE(!keep && !want_stats && !fr->mask_used && !want_t, MLPSP_E_ARG,
                  "per-pixel ordering renders rgb, alpha and the feature map only");
    MLPSP_REQUIRE(fr->tile_capacity <= kWinMax, MLPSP_E_LIMIT, "per-pixel ordering needs tile_capacity <= %d", kWinMax);
  }
  if (want_stats)
    MLPSP_REQUIRE(fr->gt_rgb && fr->stat_max_w && fr->stat_hits && fr->stat_sum_werr && fr->stat_contrib, MLPSP_E_ARG,
                  "contribution statistics need gt_rgb and all five per-primitive arrays");
  const PrimStats pstats = {fr->gt_rgb, fr->sorted_prims, fr->stat_sum_w, fr->stat_max_w, fr->stat_hits,
                            fr->stat_sum_werr, fr->stat_contrib};
  // record export reads the consumed masks from the scratch copy, so a caller-owned mask buffer is
  // filled by a device copy afterwards
  uint32_t* used32 = (keep || want_feat) ? s.used32 : (uint32_t*)fr->mask_used;
  {
    LaunchScope scope(kKMisc, 1, st);
    const int64_t span = std::max<int64_t>(std::max<int64_t>(P, T), n);
    launch_chained(k_init_frame, dim3((unsigned)((span + 255) / 256)), dim3(256), 0, st, P, s.px_state, s.px_depth, fr->rgb, fr->alpha, fr->depth_t, bg[0], bg[1],
                                                                bg[2], T, s.active[0], s.counters, fr->tile_offsets, s.tile_len,
                                                                lists_refined ? 1 : 0, n, s.prim_cnt, s.prim_cursor);
  }
  if (used32) MLPSP_CUDA_OK(cudaMemsetAsync(used32, 0, 8 * (size_t)fr->max_pairs, st));
  if (n == 0) {
    if (want_feat) MLPSP_CUDA_OK(cudaMemsetAsync(fr->feat, 0, 4 * (size_t)P * sc->feat_dim, st));
    return cuda_check(cudaGetLastError(), "render_sorted");
  }
  const bool tc_path = fr->precision == MLPSP_PRECISION_F16 || fr->precision == MLPSP_PRECISION_BF16;
  const bool ref_arith = fr->hit_arith == 1;
  // Small groups get their own work list and kernel when the tensor-core evaluator runs and the scene is one whose
  // primitives own few records each: a frame evaluates about a dozen records per pixel, so with more than one
  // primitive per three pixels the typical primitive has fewer than 40 records per frame.  With fewer primitives the
  // extra launch per wave costs more than the few remainders gain (measured: 250,000 primitives on 816,000 pixels
  // lose 4 % of evaluator time with the second list, 500,000 gain 2 %, 2,000,000 with 64 hidden units gain 21 %).  (Record export keeps one list.)
  const bool split_small = tc_path && !keep && (int64_t)n * 3 > P;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // CTAs walk the active-tile list with a grid stride, so a wave with few (or no) live tiles costs a
  // launch of a few thousand CTAs, not one per tile of the image
  const int wave_grid = std::min(T, sms * 16);
  // per-pixel ordering: one wave over the whole lists, every pixel live
  const int nw = per_pixel ? 1 : (fr->num_waves > 0 ? fr->num_waves : (int)(sizeof(kDefaultWaves) / sizeof(int)));
  int lo = 0;
  for (int w = 0; w < nw && lo < fr->tile_capacity; ++w) {
    const int wl = per_pixel ? fr->tile_capacity : (fr->num_waves > 0 ? fr->wave_len[w] : kDefaultWaves[w]);
    MLPSP_REQUIRE(wl > 0, MLPSP_E_ARG, "wave_len[%d] must be positive", w);
    int hi = (wl >= fr->tile_capacity - lo || w == nw - 1) ? fr->tile_capacity : lo + wl;
    MLPSP_REQUIRE(hi - lo <= kWinMax, MLPSP_E_LIMIT, "wave window beyond %d candidates", kWinMax);
    const int cur = w & 1, nxt = cur ^ 1;
    // a last wave the caller expects to be idle: one CTA per SM walks whatever is left
    const bool idle_tail = fr->tail_hint == 1 && hi == fr->tile_capacity && w > 0;
    const int grid_hits = idle_tail ? sms : wave_grid;
    const int grid_comp = idle_tail ? sms : std::min(T, sms * 32);
    const int cap_mlp = idle_tail ? sms : 0;
    const int32_t* act = s.active[cur];
    const int32_t* act_n = s.counters + kCtrActive0 + cur;
    { LaunchScope scope(kKHits, 1, st);
    if (ref_arith)
      launch_chained(k_hits<true>, dim3(grid_hits), dim3(256), 0, st, fr->rays_o, fr->rays_d, (const float4*)sc->geom, n, fr->tile_offsets, s.tile_len, fr->sorted_prims,
                              W, H, ntx, fr->threshold, miss_bound2(fr->threshold), act, act_n, lo, hi, s.px_state,
                              s.masks32, s.pair_base,
                              s.prim_cnt + (size_t)(w & 1) * prim_cnt_stride(n), s.counters, fr->max_records, fr->status, nullptr);
    else
      launch_chained(k_hits<false>, dim3(grid_hits), dim3(256), 0, st, fr->rays_o, fr->rays_d, (const float4*)sc->geom, n, fr->tile_offsets, s.tile_len, fr->sorted_prims,
                              W, H, ntx, fr->threshold, miss_bound2(fr->threshold), act, act_n, lo, hi, s.px_state,
                              s.masks32, s.pair_base,
                              s.prim_cnt + (size_t)(w & 1) * prim_cnt_stride(n), s.counters, fr->max_records, fr->status, nullptr); }
    int rc = launch_prim_scan(s, n, nxt, fr->status, st, split_small, w);
    if (rc) return rc;
    { LaunchScope scope(kKFill, 1, st);
    launch_chained(k_fill, dim3(grid_hits), dim3(256), 0, st, fr->rays_o, fr->rays_d, (const float4*)sc->geom, fr->tile_offsets, s.tile_len, fr->sorted_prims,
                              W, H, ntx, fr->threshold, act, act_n, lo, hi, s.masks32, s.pair_base, s.prim_off,
                              s.prim_cursor, s.rec_in, (want_t || per_pixel) ? s.rec_t : nullptr,
                              (want_feat && sc->feat_slots > 1) ? s.rec_gate : nullptr, sc->gate_beta,
                              sc->gate_tau, per_pixel ? 1 : 0, ref_arith ? 1 : 0, fr->status); }
    if (tc_path)
      rc = launch_mlp_f16(sc, s.rec_in, s.prim_off, s.work, s.counters, s.rec_out, keep ? s.rec_ext : nullptr, kOutAlpha,
                          fr->status, st, fr->precision == MLPSP_PRECISION_BF16, cap_mlp, split_small ? s.work_small : nullptr);
    else
      rc = launch_mlp_f32(sc, s.rec_in, s.prim_off, s.work, s.counters, s.rec_out, keep ? s.rec_ext : nullptr, kOutAlpha,
                          fr->status, st, cap_mlp);
    if (rc) return rc;
    if (per_pixel) {
      LaunchScope scope(kKComposite, 1, st);
      k_composite_per_pixel<<<std::min(T, sms * 32), 64, 0, st>>>(fr->tile_offsets, s.tile_len, T, W, H, ntx, s.masks32, s.pair_base,
                                                                 s.rec_out, s.rec_t, fr->rgb, fr->alpha, bg[0], bg[1], bg[2],
                                                                 has_bg, want_feat ? used32 : nullptr,
                                                                 want_feat ? s.rec_w : nullptr, fr->status);
      break;
    }
    { LaunchScope scope(kKComposite, 1, st);
    if (want_stats)
      launch_chained(k_composite<true>, dim3(grid_comp), dim3(64), 0, st, pstats, fr->tile_offsets, s.tile_len, W, H, ntx, act, act_n, lo, hi, s.masks32, s.pair_base,
                                  s.rec_out, want_t ? s.rec_t : nullptr, s.px_state, s.px_depth, fr->rgb,
                                  fr->alpha, fr->depth_t, used32, want_feat ? s.rec_w : nullptr,
                                  keep ? s.rec_tr : nullptr, bg[0], bg[1], bg[2], has_bg,
                                  s.active[nxt], s.counters + kCtrActive0 + nxt, fr->status);
    else
    launch_chained(k_composite<false>, dim3(grid_comp), dim3(64), 0, st, pstats, fr->tile_offsets, s.tile_len, W, H, ntx, act, act_n, lo, hi, s.masks32, s.pair_base,
                                  s.rec_out, want_t ? s.rec_t : nullptr, s.px_state, s.px_depth, fr->rgb,
                                  fr->alpha, fr->depth_t, used32, want_feat ? s.rec_w : nullptr,
                                  keep ? s.rec_tr : nullptr, bg[0], bg[1], bg[2], has_bg,
                                  s.active[nxt], s.counters + kCtrActive0 + nxt, fr->status); }
    lo = hi;
  }
  if (fr->mask_used && used32 != (uint32_t*)fr->mask_used)
    MLPSP_CUDA_OK(cudaMemcpyAsync(fr->mask_used, used32, 8 * (size_t)fr->max_pairs, cudaMemcpyDeviceToDevice, st));
  if (want_feat && feature_tc_supported(sc)) {
    // binary16 attributes and a channel count the tensor-core kernel takes: the contraction runs on tcgen05
    LaunchScope scope(kKComposite, 1, st);
    const int rc_ft = launch_feature_tc(sc, fr, s, used32, st);
    if (rc_ft) return rc_ft;
  } else if (want_feat) {
    static DeviceOnce attr_once;
    const int CB = std::min(sc->feat_dim, kFeatChan);
    const size_t smem = sizeof(float) * 64 * (size_t)CB;
    if (attr_once.first()) {
      MLPSP_CUDA_OK(cudaFuncSetAttribute(k_feature_composite<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * kFeatChan * 4));
      MLPSP_CUDA_OK(cudaFuncSetAttribute(k_feature_composite<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * kFeatChan * 4));
    }
    LaunchScope scope(kKComposite, 1, st);
    const dim3 grid(T, (sc->feat_dim + CB - 1) / CB);
    const bool vec = sc->feat_dim >= kFeatChan && (sc->feat_dim & 3) == 0 && (reinterpret_cast<uintptr_t>(sc->feat_attr) & 15) == 0;
    if (vec)
      k_feature_composite<true><<<grid, kFeatThreads, smem, st>>>(fr->tile_offsets, s.tile_len, fr->sorted_prims, W, H, ntx, used32, s.masks32,
                                                                 s.pair_base, s.rec_w, s.rec_gate, sc->feat_attr, sc->feat_slots,
                                                                 sc->feat_dim, CB, fr->feat, fr->status);
    else
      k_feature_composite<false><<<grid, kFeatThreads, smem, st>>>(fr->tile_offsets, s.tile_len, fr->sorted_prims, W, H, ntx, used32, s.masks32,
                                                                  s.pair_base, s.rec_w, s.rec_gate, sc->feat_attr, sc->feat_slots,
                                                                  sc->feat_dim, CB, fr->feat, fr->status);
  }
  return cuda_check(cudaGetLastError(), "render_sorted");
}

// ----------------------------------------------------------------------- view batches ----
// Several views of one scene rendered together (rgb and alpha only).  Binning, sorting, hit masks, record fill and
// compositing run per view on the view's own scratch; what is shared is everything per primitive: the record
// counts, the CSR offsets, the work list and the record arrays live in the first frame's scratch, compositing
// slots are numbered across the views, and ONE evaluator launch per wave serves all views.  A primitive's weight
// image is then fetched once per wave for the records of all views, which is what bounds many-primitive scenes
// (a few records per primitive and view).  Every record goes through the same arithmetic as in a frame rendered
// alone, so the images are bit-identical.
int launch_render_batch(const mlpsp_scene* sc, const mlpsp_frame* frs, const Scratch* ss, int V, cudaStream_t st,
                        bool lists_refined) {
  const mlpsp_frame* f0 = frs;
  const Scratch& lead = ss[0];
  const int W = f0->width, H = f0->height;
  const int T = num_tiles(W, H, 8);
  const int ntx = (W + 7) / 8;
  const int64_t P = (int64_t)W * H;
  const int n = sc->n;
  const PrimStats no_stats = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  {
    LaunchScope scope(kKMisc, V, st);
    for (int v = 0; v < V; ++v) {
      const mlpsp_frame* fr = frs + v;
      float bg[3] = {0.f, 0.f, 0.f};
      if (fr->bg_color) { bg[0] = fr->bg_color[0]; bg[1] = fr->bg_color[1]; bg[2] = fr->bg_color[2]; }
      const int nv = v == 0 ? n : 0;     // the per-primitive arrays are the first frame's
      const int64_t span = std::max<int64_t>(std::max<int64_t>(P, T), nv);
      launch_chained(k_init_frame, dim3((unsigned)((span + 255) / 256)), dim3(256), 0, st, P, ss[v].px_state, ss[v].px_depth, fr->rgb, fr->alpha, nullptr, bg[0], bg[1],
                                                                  bg[2], T, ss[v].active[0], ss[v].counters, fr->tile_offsets,
                                                                  ss[v].tile_len, lists_refined ? 1 : 0, nv, lead.prim_cnt, lead.prim_cursor);
    }
  }
  if (n == 0) return cuda_check(cudaGetLastError(), "render_batch");
  const bool tc_path = f0->precision == MLPSP_PRECISION_F16 || f0->precision == MLPSP_PRECISION_BF16;
  const bool ref_arith = f0->hit_arith == 1;
  // the second work list costs one launch per wave and batch, not per view, so it pays earlier than for one frame
  // (measured with and without: fourview_500k in one batch of 4 views 2.51 -> 2.31 ms, stress_2m in batches of 16
  // views 72.2 -> 65.8 ms of evaluator time)
  const bool split_small = tc_path && (int64_t)n * 20 > P * V;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int wave_grid = std::min(T, sms * 16);
  const int nw = f0->num_waves > 0 ? f0->num_waves : (int)(sizeof(kDefaultWaves) / sizeof(int));
  int lo = 0;
  for (int w = 0; w < nw && lo < f0->tile_capacity; ++w) {
    const int wl = f0->num_waves > 0 ? f0->wave_len[w] : kDefaultWaves[w];
    MLPSP_REQUIRE(wl > 0, MLPSP_E_ARG, "wave_len[%d] must be positive", w);
    const int hi = (wl >= f0->tile_capacity - lo || w == nw - 1) ? f0->tile_capacity : lo + wl;
    MLPSP_REQUIRE(hi - lo <= kWinMax, MLPSP_E_LIMIT, "wave window beyond %d candidates", kWinMax);
    const int cur = w & 1, nxt = cur ^ 1;
    const bool idle_tail = f0->tail_hint == 1 && hi == f0->tile_capacity && w > 0;
    const int grid_hits = idle_tail ? sms : wave_grid;
    const int grid_comp = idle_tail ? sms : std::min(T, sms * 32);
    const int cap_mlp = idle_tail ? sms : 0;
    int32_t* cnt = lead.prim_cnt + (size_t)(w & 1) * prim_cnt_stride(n);
    {
      LaunchScope scope(kKHits, V, st);
      for (int v = 0; v < V; ++v) {
        const mlpsp_frame* fr = frs + v;
        const Scratch& s = ss[v];
        if (ref_arith)
          launch_chained(k_hits<true>, dim3(grid_hits), dim3(256), 0, st, fr->rays_o, fr->rays_d, (const float4*)sc->geom, n, fr->tile_offsets, s.tile_len,
                                                  fr->sorted_prims, W, H, ntx, f0->threshold, miss_bound2(f0->threshold), s.active[cur],
                                                  s.counters + kCtrActive0 + cur, lo, hi, s.px_state, s.masks32, s.pair_base, cnt,
                                                  lead.counters, f0->max_records, f0->status, s.counters + kCtrActive0 + nxt);
        else
          launch_chained(k_hits<false>, dim3(grid_hits), dim3(256), 0, st, fr->rays_o, fr->rays_d, (const float4*)sc->geom, n, fr->tile_offsets, s.tile_len,
                                                   fr->sorted_prims, W, H, ntx, f0->threshold, miss_bound2(f0->threshold), s.active[cur],
                                                   s.counters + kCtrActive0 + cur, lo, hi, s.px_state, s.masks32, s.pair_base, cnt,
                                                   lead.counters, f0->max_records, f0->status, s.counters + kCtrActive0 + nxt);
      }
    }
    int rc = launch_prim_scan(lead, n, nxt, f0->status, st, split_small, w);
    if (rc) return rc;
    {
      LaunchScope scope(kKFill, V, st);
      for (int v = 0; v < V; ++v) {
        const mlpsp_frame* fr = frs + v;
        const Scratch& s = ss[v];
        launch_chained(k_fill, dim3(grid_hits), dim3(256), 0, st, fr->rays_o, fr->rays_d, (const float4*)sc->geom, fr->tile_offsets, s.tile_len, fr->sorted_prims,
                                          W, H, ntx, f0->threshold, s.active[cur], s.counters + kCtrActive0 + cur, lo, hi, s.masks32,
                                          s.pair_base, lead.prim_off, lead.prim_cursor, lead.rec_in, nullptr, nullptr, sc->gate_beta,
                                          sc->gate_tau, 0, ref_arith ? 1 : 0, f0->status);
      }
    }
    if (tc_path)
      rc = launch_mlp_f16(sc, lead.rec_in, lead.prim_off, lead.work, lead.counters, lead.rec_out, nullptr, kOutAlpha, f0->status, st,
                          f0->precision == MLPSP_PRECISION_BF16, cap_mlp, split_small ? lead.work_small : nullptr);
    else
      rc = launch_mlp_f32(sc, lead.rec_in, lead.prim_off, lead.work, lead.counters, lead.rec_out, nullptr, kOutAlpha, f0->status, st, cap_mlp);
    if (rc) return rc;
    {
      LaunchScope scope(kKComposite, V, st);
      for (int v = 0; v < V; ++v) {
        const mlpsp_frame* fr = frs + v;
        const Scratch& s = ss[v];
        float bg[3] = {0.f, 0.f, 0.f};
        const int has_bg = fr->bg_color != nullptr;
        if (has_bg) { bg[0] = fr->bg_color[0]; bg[1] = fr->bg_color[1]; bg[2] = fr->bg_color[2]; }
        launch_chained(k_composite<false>, dim3(grid_comp), dim3(64), 0, st, no_stats, fr->tile_offsets, s.tile_len, W, H, ntx, s.active[cur],
                                                     s.counters + kCtrActive0 + cur, lo, hi, s.masks32, s.pair_base, lead.rec_out, nullptr,
                                                     s.px_state, s.px_depth, fr->rgb, fr->alpha, nullptr, nullptr, nullptr, nullptr, bg[0],
                                                     bg[1], bg[2], has_bg, s.active[nxt], s.counters + kCtrActive0 + nxt, f0->status);
      }
    }
    lo = hi;
  }
  return cuda_check(cudaGetLastError(), "render_batch");
}

// ----------------------------------------------------------------------- record export ----
// Pixel-major records in compositing order (np_tile_kernels.cu:3138-3154; training_wmma.cuh:223-256),
// rebuilt after the frame from the consumed masks, the evaluator outputs kept per compositing slot
// and a recomputed hit test.  Two passes like the reference: count per pixel, prefix, emit.
template <bool EMIT>
__global__ void __launch_bounds__(64) k_export(
    const float* __restrict__ rays_o, const float* __restrict__ rays_d, const float4* __restrict__ geom,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, const int32_t* __restrict__ sorted_prims, int W, int H, int ntx,
    float thr, float beta, float tau, const uint32_t* __restrict__ used32, const uint32_t* __restrict__ masks32,
    const uint32_t* __restrict__ pair_base, const float4* __restrict__ rec_out, const float4* __restrict__ rec_ext,
    const float* __restrict__ rec_tr, const float4* __restrict__ px_state, int32_t* __restrict__ px_cnt,
    const int32_t* __restrict__ px_off, int max_hits, int32_t* __restrict__ worst, int32_t* __restrict__ ids,
    float* __restrict__ x6, float* __restrict__ raw, int32_t* __restrict__ relu_masks, float* __restrict__ gates,
    int64_t max_out, int ref_arith, const int32_t* __restrict__ status) {
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tile = blockIdx.x;
  const int s = tile_offsets[tile], e = s + tile_len[tile];
  const int lane = threadIdx.x & 31, half = threadIdx.x >> 5;
  const TilePix tp = tile_pixel(tile, half * 32 + lane, ntx, W, H);
  V3 o = {0.f, 0.f, 0.f}, d = {0.f, 0.f, 0.f};
  int64_t out0 = 0;
  if (EMIT && tp.valid) { o = load3(rays_o, tp.pix); d = load3(rays_d, tp.pix); out0 = px_off[tp.pix]; }
  const uint32_t lt = (1u << lane) - 1u;
  int cnt = 0;
  for (int i0 = s; i0 < e; i0 += 32) {
    const int idx = i0 + lane;
    uint2 uu = make_uint2(0u, 0u);
    if (idx < e) uu = *reinterpret_cast<const uint2*>(used32 + 2 * (size_t)idx);
    const uint32_t any = __ballot_sync(0xffffffffu, (half ? uu.y : uu.x) != 0u);
    if (!EMIT) {
      // count: bit `lane` of every pair's half mask
      uint32_t pending = any;
      while (pending) {
        const int j = __ffs(pending) - 1;
        pending &= pending - 1;
        const uint32_t mine = __shfl_sync(0xffffffffu, half ? uu.y : uu.x, j);
        cnt += (mine >> lane) & 1u;
      }
      continue;
    }
    uint32_t pending = any;
    while (pending) {
      const int j = __ffs(pending) - 1;
      pending &= pending - 1;
      const uint32_t mine = __shfl_sync(0xffffffffu, half ? uu.y : uu.x, j);
      if (!((mine >> lane) & 1u)) continue;
      const int i = i0 + j;
      const uint32_t m0 = masks32[2 * (size_t)i], m1 = masks32[2 * (size_t)i + 1];
      const uint32_t hitm = half ? m1 : m0;
      const uint32_t slot = pair_base[i] + (half ? __popc(m0) : 0) + __popc(hitm & lt);
      const int p = sorted_prims[i];
      const int64_t r = out0 + cnt;
      ++cnt;
      if (r >= max_out) continue;
      Hit h;
      if (ref_arith) hit_test_ref(load_geom_ref(geom, p), o, d, thr, h);
      else hit_test(load_geom(geom, p), o, d, thr, h);
      if (ids) ids[r] = p;
      if (x6) { float* q = x6 + r * 6; q[0] = d.x; q[1] = d.y; q[2] = d.z; q[3] = h.dx; q[4] = h.dy; q[5] = h.dz; }
      const float4 ro = rec_out[slot], re = rec_ext[slot];
      if (raw) {
        float* q = raw + r * 8;
        q[0] = ro.x; q[1] = ro.y; q[2] = ro.z; q[3] = re.x; q[4] = rec_tr[slot]; q[5] = ro.w; q[6] = h.decay; q[7] = re.y;
      }
      if (relu_masks) { relu_masks[r * 2] = (int32_t)__float_as_uint(re.z); relu_masks[r * 2 + 1] = (int32_t)__float_as_uint(re.w); }
      if (gates) {
        const float4 ls = __ldg(geom + (size_t)p * 4 + 3);
        const float4 g = tetra_gates(h, ls.x, ls.y, ls.z, beta, tau);
        float* q = gates + r * 4; q[0] = g.x; q[1] = g.y; q[2] = g.z; q[3] = g.w;
      }
    }
  }
  if (!EMIT && tp.valid) {
    px_cnt[tp.pix] = cnt;
    atomicMax(worst, cnt);
    const bool live = px_state[tp.pix].w >= MLPSP_TERM;
    if (max_hits > 0 && cnt >= max_hits && (cnt > max_hits || live)) atomicOr(worst + 1, 1);
  }
}

__global__ void k_widen_i32(const int32_t* __restrict__ in, int64_t n, int64_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[i];
}

int launch_export_records(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, int64_t* offsets, int32_t* ids,
                          float* x6, float* raw, int32_t* relu_masks, float* gates, int64_t max_out, int32_t max_hits,
                          int64_t* total_host, int32_t* worst_host, cudaStream_t st) {
  const int W = fr->width, H = fr->height, T = num_tiles(W, H, 8), ntx = (W + 7) / 8;
  const int64_t P = (int64_t)W * H;
  int32_t* worst = s.counters + kCtrScratch;     // [0] largest per-pixel count, [1] capacity flag
  MLPSP_CUDA_OK(cudaMemsetAsync(worst, 0, 8, st));
  LaunchScope scope(kKMisc, 3 + scan_launches(P), st);
  k_export<false><<<T, 64, 0, st>>>(fr->rays_o, fr->rays_d, (const float4*)sc->geom, fr->tile_offsets, s.tile_len, fr->sorted_prims,
                                    W, H, ntx, fr->threshold, sc->gate_beta, sc->gate_tau, s.used32, s.masks32,
                                    s.pair_base, s.rec_out, s.rec_ext, s.rec_tr, s.px_state, s.px_cnt, nullptr, max_hits,
                                    worst, nullptr, nullptr, nullptr, nullptr, nullptr, 0, fr->hit_arith == 1 ? 1 : 0, fr->status);
  int rc = launch_scan_i32(s.px_cnt, P, s.scan_blk, s.px_off, st);
  if (rc) return rc;
  k_widen_i32<<<(unsigned)((P + 1 + 255) / 256), 256, 0, st>>>(s.px_off, P + 1, offsets);
  int32_t h[3] = {0, 0, 0};
  MLPSP_CUDA_OK(cudaMemcpyAsync(&h[0], s.px_off + P, 4, cudaMemcpyDeviceToHost, st));
  MLPSP_CUDA_OK(cudaMemcpyAsync(&h[1], worst, 8, cudaMemcpyDeviceToHost, st));
  MLPSP_CUDA_OK(cudaStreamSynchronize(st));
  if (total_host) *total_host = h[0];
  if (worst_host) *worst_host = h[2] ? -h[1] : h[1];
  if ((ids || x6 || raw || relu_masks || gates) && max_out >= h[0] && h[0] > 0) {
    k_export<true><<<T, 64, 0, st>>>(fr->rays_o, fr->rays_d, (const float4*)sc->geom, fr->tile_offsets, s.tile_len, fr->sorted_prims,
                                     W, H, ntx, fr->threshold, sc->gate_beta, sc->gate_tau, s.used32, s.masks32,
                                     s.pair_base, s.rec_out, s.rec_ext, s.rec_tr, s.px_state, s.px_cnt, s.px_off, max_hits,
                                     worst, ids, x6, raw, relu_masks, gates, max_out, fr->hit_arith == 1 ? 1 : 0, fr->status);
  }
  return cuda_check(cudaGetLastError(), "export_records");
}

}  // namespace mlpsp
