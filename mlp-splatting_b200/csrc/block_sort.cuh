// Stable block-wide LSD radix sort of up to CAP (key, value) pairs held in shared memory.
//
// 4-bit digits.  Each warp walks chunks of 32 consecutive items; inside a chunk the rank of an
// item among equal digits comes from match.any + popc (lane order = list order, so the pass is
// stable); per-(digit, chunk) counts are scanned digit-major to give scatter bases.  Digit
// positions whose bits are equal across the whole list are skipped.
#pragma once
#include "common.cuh"

namespace mlpsp {

template <int THREADS, int CAP>
struct BlockRadixSort {
  static constexpr int kChunks = CAP / 32;
  static constexpr int kBins = 16;
  struct Smem {
    uint32_t key[2][CAP];
    int32_t val[2][CAP];
    int32_t cnt[kBins * kChunks];
    int32_t warp_sums[32];
    uint32_t red[THREADS / 32];
  };

  // Sorts items [0,n) of buffer 0 ascending by key (stable).  Returns the buffer index that holds
  // the result.  All threads of the block must call it; ends with a barrier.
  __device__ static int sort(Smem& s, const int n) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = THREADS / 32;
    const int nchunks = (n + 31) >> 5;
    // which bit positions vary at all
    uint32_t diff = 0;
    const uint32_t k0 = s.key[0][0];
    for (int i = tid; i < n; i += THREADS) diff |= s.key[0][i] ^ k0;
    diff = __reduce_or_sync(0xffffffffu, diff);
    if (lane == 0) s.red[warp] = diff;
    __syncthreads();
    diff = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) diff |= s.red[w];
    int cur = 0;
    for (int shift = 0; shift < 32; shift += 4) {
      if (((diff >> shift) & 15u) == 0u) continue;
      const int ncnt = kBins * nchunks;
      for (int i = tid; i < ncnt; i += THREADS) s.cnt[i] = 0;
      __syncthreads();
      for (int c = warp; c < nchunks; c += NW) {
        const int i = c * 32 + lane;
        const bool valid = i < n;
        const uint32_t d = valid ? ((s.key[cur][i] >> shift) & 15u) : 0xffffffffu;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        if (valid && lane == __ffs(peers) - 1) s.cnt[d * nchunks + c] = __popc(peers);
      }
      __syncthreads();
      // exclusive scan of cnt[0, ncnt) in index order (digit-major, chunk-minor)
      const int per = (ncnt + THREADS - 1) / THREADS;
      const int b = tid * per;
      int local = 0;
      for (int j = 0; j < per; ++j) if (b + j < ncnt) local += s.cnt[b + j];
      int total;
      int base = block_exclusive_scan(local, s.warp_sums, total);
      for (int j = 0; j < per; ++j)
        if (b + j < ncnt) { const int v = s.cnt[b + j]; s.cnt[b + j] = base; base += v; }
      __syncthreads();
      for (int c = warp; c < nchunks; c += NW) {
        const int i = c * 32 + lane;
        const bool valid = i < n;
        const uint32_t k = valid ? s.key[cur][i] : 0u;
        const uint32_t d = valid ? ((k >> shift) & 15u) : 0xffffffffu;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        if (valid) {
          const int dst = s.cnt[d * nchunks + c] + __popc(peers & ((1u << lane) - 1u));
          s.key[cur ^ 1][dst] = k;
          s.val[cur ^ 1][dst] = s.val[cur][i];
        }
      }
      __syncthreads();
      cur ^= 1;
    }
    return cur;
  }
};

}  // namespace mlpsp
