// Feature decoder and text query: the step that follows the feature map.
//
// The reference decodes a low-dimensional rendered feature map with a three-layer convolutional
// network (1x1 -> ReLU -> 3x3, zero padding 1 -> ReLU -> 1x1; scannet/feature_decoder.py:5-19, called at
// scannet/eval_lseg_table2.py:1221-1225), L2-normalises the result, multiplies it with the normalised
// text embeddings and takes the arg-max class per pixel (eval_lseg_table2.py:622-641).  With a 512-wide
// output that is a 1.67 GB map per 1200x680 frame that exists only to be reduced to one label per pixel.
//
// k_decode_tc runs the whole chain per tile of 8 x 16 output pixels on the tensor cores (tcgen05,
// FP32 accumulators in tensor memory, binary16 operands as in the MLP evaluator):
//   layer 1  D1[180 x Ch] = X[180 x Cin] . W1^T for the tile and its one-pixel halo (two M = 128 MMAs that
//            overlap on rows 52..127), bias + ReLU, halo pixels outside the image forced to zero (they are
//            the 3x3 convolution's zero padding);
//   layer 2  nine taps, each a [128 x Ch] . [Ch x Ch] product whose A operand is the SAME hidden tile in
//            shared memory addressed through a shifted descriptor: with the tile 8 pixels wide, one halo
//            row is one core-matrix group (8 rows of 16 bytes, consecutive), groups are 160 bytes apart
//            (10 halo pixels) and a tap (ty, tx) only moves the start address by (10 ty + tx) * 16 bytes;
//   layer 3  either the 1x1 output convolution (decoded features written out), or -- for a text query --
//            the product with M = T^ W3 folded at pack time: arg-max_c t^_c . (W3 h + b3) / |..| equals
//            arg-max_c (M h + T^ b3)_c because the normalisation is one positive factor per pixel, so the
//            wide feature vector is never formed.
// Weight blocks (W1, the nine taps, the output chunks; <= 32 KB each) stream from the packed image (L2
// resident) through a three-deep ring of bulk copies; a block's buffer is released by the commit of the MMAs
// that read it.  While the issuing lane walks the nine taps the other warps fetch the next tile's input.  One
// CTA per SM (225 KB of shared memory, all 512 tensor-memory columns).
//
// Every wait on an mbarrier is bounded; when one gives up the CTA raises MLPSP_ST_TIMEOUT, waits
// (bounded) for its own copies in flight, frees its tensor memory and returns.
#include "frame.cuh"
#include "tc.cuh"

#include <algorithm>

namespace mlpsp {

constexpr int kDecTileW = 8, kDecTileH = 16;                       // 128 output pixels = MMA M
constexpr int kHaloW = kDecTileW + 2, kHaloH = kDecTileH + 2;
constexpr int kHaloPx = kHaloW * kHaloH;                           // 180
constexpr int kDecThreads = 256;
constexpr int kColGroups = kDecThreads / 128;                        // warps that share a tensor-memory lane quarter split the columns
constexpr int kDecBlock = 32768;                                   // one weight block: <= 128 x 128 halves
constexpr int kDecRing = 3;
constexpr int kStageFloats = 32 * 32;                               // one warp's output staging tile: 32 pixels x 32 columns, 16-byte units XOR-swizzled by pixel
constexpr int kDecPieces = 8;                                      // bulk copies per weight block (block sizes are multiples of 1 KB)
constexpr int kDecSub = 1;                                         // tiles that share one pass over the weights
constexpr int kDecMaxBlocks = 16;                                  // per pass: W1, 9 taps, <= 6 output chunks
constexpr int kDecMaxDim = 128;                                    // input and hidden width limit
constexpr int kDecMaxOut = 768;

struct DecHeader {                      // first 256 bytes of the packed image
  int32_t magic, in_dim, k1, hidden, n_out, n_pad, mode, num_blocks;
  int32_t blk_off[kDecMaxBlocks], blk_bytes[kDecMaxBlocks];
  int32_t bias_off, total_bytes;
  int32_t pad[22];
};
static_assert(sizeof(DecHeader) == 256, "packed decoder header");
constexpr int32_t kDecMagic = 0x44454331;

// shared-memory plan (bytes)
constexpr int kDecH1Bytes = (kDecMaxDim / 8) * kHaloPx * 16;          // 46,080: one hidden tile with halo
constexpr int kSmRing = 0;
constexpr int kSmA0 = kSmRing + kDecRing * kDecBlock;                 //  98,304
constexpr int kA0Pitch = kHaloPx + 1;                                 // 16-byte units between K chunks of the input tile (odd)
constexpr int kSmH1 = kSmA0 + (kDecMaxDim / 8) * kA0Pitch * 16;       // +46,336
constexpr int kSmBias = kSmH1 + kDecSub * kDecH1Bytes;                // +46,080
constexpr int kSmHdr = kSmBias + 4 * (2 * kDecMaxDim + kDecMaxOut);   // + 4,096
constexpr int kSmBar = kSmHdr + 256;
constexpr int kSmMisc = kSmBar + 16 * 8;
constexpr int kSmArg = kSmMisc + 64;                                  // [2][128] (value, index) pairs
constexpr int kSmStage = kSmArg + kDecSub * kColGroups * 128 * 8;     // output staging tiles of the first eight warps
constexpr int kDecSmem = kSmStage + 8 * kStageFloats * 4;
static_assert(kDecSmem <= 227 * 1024, "shared memory of the decoder");

static int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Layout of the packed image for a decoder; false when the sizes are outside the kernel's limits.
static bool dec_layout(const mlpsp_decoder* d, int mode, DecHeader* h) {
  memset(h, 0, sizeof(*h));
  if (d->in_dim < 1 || d->in_dim > kDecMaxDim || d->hidden < 32 || d->hidden > kDecMaxDim || d->hidden % 32) return false;
  const int n_out = mode == 1 ? d->num_classes : d->out_dim;
  if (n_out < 1 || n_out > kDecMaxOut || d->out_dim < 1) return false;
  h->magic = kDecMagic;
  h->in_dim = d->in_dim;
  h->k1 = round_up(d->in_dim, 16);
  h->hidden = d->hidden;
  h->n_out = n_out;
  h->n_pad = round_up(n_out, 32);
  h->mode = mode;
  int off = 256, nb = 0;
  h->blk_off[nb] = off; h->blk_bytes[nb] = h->k1 * d->hidden * 2; off += h->blk_bytes[nb++];
  for (int t = 0; t < 9; ++t) { h->blk_off[nb] = off; h->blk_bytes[nb] = d->hidden * d->hidden * 2; off += h->blk_bytes[nb++]; }
  for (int c = 0; c * 128 < h->n_pad; ++c) {
    const int nc = std::min(128, h->n_pad - c * 128);
    h->blk_off[nb] = off; h->blk_bytes[nb] = d->hidden * nc * 2; off += h->blk_bytes[nb++];
  }
  h->num_blocks = nb;
  h->bias_off = off;
  off += 4 * (2 * d->hidden + h->n_pad);
  h->total_bytes = round_up(off, 256);
  return nb <= kDecMaxBlocks;
}

// either half of a packed binary16 pair is inf or NaN
__device__ __forceinline__ bool h2_nonfinite(uint32_t w) { return (w & 0x7c00u) == 0x7c00u || ((w >> 16) & 0x7c00u) == 0x7c00u; }

__device__ __forceinline__ uint16_t to_h16(float x, bool& bad) {
  const __half v = __float2half_rn(x);
  bad |= __hisinf(v) || __hisnan(v);
  return *reinterpret_cast<const uint16_t*>(&v);
}

// Fill the weight blocks and the bias block.  B operands are K-major core matrices: element (n, k) of a block
// with N rows sits at half index (k / 8) * N * 8 + n * 8 + k % 8.
// mode 1: folded[c][k] = sum_j t^[c][j] W3[j][k] and fb[c] = sum_j t^[c][j] b3[j] were prepared by k_fold_text.
__global__ void k_pack_decoder(DecHeader h, const float* __restrict__ W1, const float* __restrict__ b1,
                               const float* __restrict__ W2, const float* __restrict__ b2,
                               const float* __restrict__ W3, const float* __restrict__ b3,
                               const float* __restrict__ folded, const float* __restrict__ fb,
                               char* __restrict__ out, int32_t* __restrict__ status) {
  const int Ch = h.hidden, Cin = h.in_dim;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x, t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool bad = false;
  uint16_t* w1 = reinterpret_cast<uint16_t*>(out + h.blk_off[0]);
  for (int64_t i = t0; i < (int64_t)Ch * h.k1; i += stride) {
    const int n = (int)(i / h.k1), k = (int)(i % h.k1);
    w1[(k >> 3) * Ch * 8 + n * 8 + (k & 7)] = to_h16(k < Cin ? W1[(int64_t)n * Cin + k] : 0.f, bad);
  }
  for (int64_t i = t0; i < (int64_t)9 * Ch * Ch; i += stride) {
    const int tap = (int)(i / (Ch * Ch)), n = (int)(i / Ch % Ch), k = (int)(i % Ch);
    uint16_t* w2 = reinterpret_cast<uint16_t*>(out + h.blk_off[1 + tap]);
    w2[(k >> 3) * Ch * 8 + n * 8 + (k & 7)] = to_h16(W2[((int64_t)n * Ch + k) * 9 + tap], bad);
  }
  for (int64_t i = t0; i < (int64_t)h.n_pad * Ch; i += stride) {
    const int n = (int)(i / Ch), k = (int)(i % Ch);
    const int c = n >> 7, nl = n & 127, nc = min(128, h.n_pad - c * 128);
    float v = 0.f;
    if (n < h.n_out) v = h.mode == 1 ? folded[(int64_t)n * Ch + k] : W3[(int64_t)n * Ch + k];
    uint16_t* w3 = reinterpret_cast<uint16_t*>(out + h.blk_off[10 + c]);
    w3[(k >> 3) * nc * 8 + nl * 8 + (k & 7)] = to_h16(v, bad);
  }
  float* bias = reinterpret_cast<float*>(out + h.bias_off);
  for (int64_t i = t0; i < 2 * Ch + h.n_pad; i += stride) {
    float v = 0.f;
    if (i < Ch) v = b1[i];
    else if (i < 2 * Ch) v = b2[i - Ch];
    else if (i - 2 * Ch < h.n_out) v = h.mode == 1 ? fb[i - 2 * Ch] : b3[i - 2 * Ch];
    bad |= !isfinite(v);
    bias[i] = v;
  }
  if (t0 == 0) *reinterpret_cast<DecHeader*>(out) = h;
  if (bad && status) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
}

// One block per class: t^ = text / max(|text|, 1e-12); folded[c][:] = t^ W3, fb[c] = t^ . b3.
__global__ void k_fold_text(const float* __restrict__ text, const float* __restrict__ W3, const float* __restrict__ b3,
                            int out_dim, int Ch, float* __restrict__ folded, float* __restrict__ fb) {
  extern __shared__ float s_t[];      // [out_dim] normalised text row, then one slot for the reduction
  __shared__ float s_red[32];
  const int c = blockIdx.x;
  float ss = 0.f;
  for (int j = threadIdx.x; j < out_dim; j += blockDim.x) { const float v = text[(int64_t)c * out_dim + j]; s_t[j] = v; ss += v * v; }
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_red[w];
  const float inv = 1.0f / fmaxf(sqrtf(tot), 1e-12f);
  for (int k = threadIdx.x; k < Ch; k += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < out_dim; ++j) acc = fmaf(s_t[j] * inv, W3[(int64_t)j * Ch + k], acc);
    folded[(int64_t)c * Ch + k] = acc;
  }
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int j = 0; j < out_dim; ++j) acc = fmaf(s_t[j] * inv, b3[j], acc);
    fb[c] = acc;
  }
}

// ---------------------------------------------------------------------------- the decoder ----

// Input tile with halo -> binary16 A operand [K1/8][kA0Pitch][8] in shared memory.  Consecutive lanes take
// consecutive 32-byte pieces of a pixel's feature row (coalesced); the odd pitch spreads the 16-byte stores
// of one pixel's chunks over all banks.  Loads are issued four units ahead of their conversion.
// Threads t = 0..nthr-1 of the CTA share the tile.
__device__ __forceinline__ bool load_input_tile(const float* __restrict__ feat, int W, int H, int Cin, int K1,
                                                int ty0, int tx0, char* s_a0, int t, int nthr) {
  // unit u = (halo pixel r, 16-byte chunk kc), chunk fastest; the chunk count is padded to a power of two so that
  // the split is a shift and a mask
  const int nk = K1 >> 3, lg = nk > 8 ? 4 : (nk > 4 ? 3 : (nk > 2 ? 2 : 1)), units = kHaloPx << lg;
  const bool vec = (Cin & 7) == 0;
  bool bad = false;
  for (int u0 = t; u0 < units; u0 += 4 * nthr) {
    float4 lo[4], hi[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int u = u0 + b * nthr;
      lo[b] = hi[b] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (u < units) {
        const int r = u >> lg, kc = u & ((1 << lg) - 1);
        const int hy = r / kHaloW, hx = r - hy * kHaloW;
        const int y = ty0 + hy - 1, x = tx0 + hx - 1;
        if (y >= 0 && y < H && x >= 0 && x < W && kc * 8 < Cin) {   // kc >= nk lies beyond Cin as well
          const float* src = feat + ((int64_t)y * W + x) * Cin + kc * 8;
          if (vec) {
            lo[b] = __ldg(reinterpret_cast<const float4*>(src));
            hi[b] = __ldg(reinterpret_cast<const float4*>(src) + 1);
          } else {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = kc * 8 + e < Cin ? __ldg(src + e) : 0.f;
            lo[b] = make_float4(v[0], v[1], v[2], v[3]);
            hi[b] = make_float4(v[4], v[5], v[6], v[7]);
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int u = u0 + b * nthr;
      const int r = u >> lg, kc = u & ((1 << lg) - 1);
      if (u < units && kc < nk) {
        uint4 w;
        w.x = pack_h2<false>(lo[b].x, lo[b].y); w.y = pack_h2<false>(lo[b].z, lo[b].w);
        w.z = pack_h2<false>(hi[b].x, hi[b].y); w.w = pack_h2<false>(hi[b].z, hi[b].w);
        bad |= h2_nonfinite(w.x) || h2_nonfinite(w.y) || h2_nonfinite(w.z) || h2_nonfinite(w.w);   // beyond binary16 range
        *reinterpret_cast<uint4*>(s_a0 + (kc * kA0Pitch + r) * 16) = w;
      }
    }
  }
  return bad;
}

// +bias, ReLU, binary16: 32 accumulator columns -> four 16-byte units of the next A operand
__device__ __forceinline__ bool relu_pack(const uint32_t (&acc)[32], const float* bias, int j, uint4& out) {
  uint32_t w[4];
  bool bad = false;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    w[e] = pack_h2_relu<false>(__uint_as_float(acc[j * 8 + e * 2]) + bias[j * 8 + e * 2],
                               __uint_as_float(acc[j * 8 + e * 2 + 1]) + bias[j * 8 + e * 2 + 1]);
    bad |= h2_nonfinite(w[e]);
  }
  out = make_uint4(w[0], w[1], w[2], w[3]);
  return bad;
}

// n MMAs D (+)= A_k . B_k whose operand descriptors advance by fixed steps (in 16-byte units of the start-address
// field).  The issuing thread is a single lane: everything it computes per MMA delays the next one, so the
// descriptors are built once per chain.
__device__ __forceinline__ void mma_chain(uint32_t d, uint64_t a, uint64_t b, uint32_t a_step, uint32_t b_step, int n,
                                          uint32_t idesc, bool accumulate_first) {
  uint32_t acc = accumulate_first ? 1u : 0u;
  for (int k = 0; k < n; ++k) {
    mma_f16(d, a, b, idesc, acc);
    a += a_step;
    b += b_step;
    acc = 1u;
  }
}

__global__ void __launch_bounds__(kDecThreads, 1) k_decode_tc(
    const char* __restrict__ image, const float* __restrict__ feat, int W, int H, int tiles_x, int num_tiles,
    float* __restrict__ out, long long* __restrict__ labels, int32_t* __restrict__ status) {
  extern __shared__ __align__(128) char smem[];
  const DecHeader& hd = *reinterpret_cast<const DecHeader*>(smem + kSmHdr);
  float* s_bias = reinterpret_cast<float*>(smem + kSmBias);
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + kSmBar);   // [0..1] full, [2..3] empty, [4] mma, [5] output chunk
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(smem + kSmMisc);
  float2* s_arg = reinterpret_cast<float2*>(smem + kSmArg);
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int num_pairs = (num_tiles + kDecSub - 1) / kDecSub;
  if ((int)blockIdx.x >= num_pairs) return;          // leave before touching tensor memory
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = warp & 3, hsel = warp >> 2;           // tensor-memory lane quarter, column interleave
  if (tid < 64) reinterpret_cast<int32_t*>(smem + kSmHdr)[tid] = __ldg(reinterpret_cast<const int32_t*>(image) + tid);
  __syncthreads();
  const int Cin = hd.in_dim, K1 = hd.k1, Ch = hd.hidden, n_out = hd.n_out, n_pad = hd.n_pad, NB = hd.num_blocks;
  const bool classify = hd.mode == 1;
  {
    const float* gb = reinterpret_cast<const float*>(image + hd.bias_off);
    for (int i = tid; i < 2 * Ch + n_pad; i += kDecThreads) s_bias[i] = __ldg(gb + i);
  }
  const uint32_t ring = smem_u32(smem + kSmRing), a0 = smem_u32(smem + kSmA0), h1 = smem_u32(smem + kSmH1);
  const uint32_t bar_full = smem_u32(&s_bar[0]), bar_empty = smem_u32(&s_bar[kDecRing]);
  const uint32_t bar_m = smem_u32(&s_bar[2 * kDecRing]), bar_o = smem_u32(&s_bar[2 * kDecRing + 1]);
  if (tid == 0) {
    for (int i = 0; i < 2 * kDecRing + 2; ++i) mbar_init(smem_u32(&s_bar[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_misc[0]), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
  const int n_my = (num_pairs - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int total_blocks = n_my * NB;
  const int out_chunks = (n_pad + 127) >> 7;
  const uint32_t idesc_h = instr_desc(128, Ch);
  static_assert(kDecSub == 1, "the early fetch of the next input assumes one tile per pass");
  const bool prefetch = true;
  int issued = 0, landed = 0;            // issuing thread only: copies requested / copies waited for
  uint32_t ph_m = 0, ph_o = 0;
  bool ok = true, bad = false;

  // issuing thread: request the copies of blocks issued..upto (ring order), each after the MMAs that read
  // the buffer's previous block have committed
  auto request = [&](int upto) {
    while (ok && issued <= upto && issued < total_blocks) {
      const int j = issued, b = j % kDecRing, use = j / kDecRing, blk = j % NB;
      if (use > 0 && !mbar_wait(bar_empty + 8 * b, (uint32_t)((use - 1) & 1))) { ok = false; break; }
      // one bulk copy moves about 12 bytes per clock; eight pieces in flight share the barrier's byte count
      const uint32_t bytes = (uint32_t)hd.blk_bytes[blk], piece = bytes / kDecPieces;
      mbar_expect_tx(bar_full + 8 * b, bytes);
      for (int pc = 0; pc < kDecPieces; ++pc)
        bulk_g2s(ring + b * kDecBlock + pc * piece, image + hd.blk_off[blk] + pc * piece, piece, bar_full + 8 * b);
      ++issued;
    }
  };
  // issuing thread: wait for block g (requested here at the latest)
  auto acquire = [&](int g) -> uint32_t {
    request(g);
    const int b = g % kDecRing;
    if (ok && !mbar_wait(bar_full + 8 * b, (uint32_t)((g / kDecRing) & 1))) ok = false;
    if (ok) landed = g + 1;
    tc_fence_after();
    return ring + b * kDecBlock;
  };
  // issuing thread: the MMAs that read block g have been issued: their commit frees the buffer, and the copies
  // that fit behind them are requested (the buffer of the block before g is free by then or very soon)
  auto release = [&](int g) {
    mma_commit(bar_empty + 8 * (g % kDecRing));
    request(g + kDecRing - 1);
  };

  for (int it = 0; it < n_my; ++it) {
    const int pair = (int)blockIdx.x + it * (int)gridDim.x;
    const int gbase = it * NB;
    int ty0[kDecSub], tx0[kDecSub];
#pragma unroll
    for (int sb = 0; sb < kDecSub; ++sb) {
      const int tile = pair * kDecSub + sb;
      // a tile past the end sits below the image: its loads give zeros and its stores are skipped
      ty0[sb] = tile < num_tiles ? (tile / tiles_x) * kDecTileH : H;
      tx0[sb] = tile < num_tiles ? (tile % tiles_x) * kDecTileW : 0;
    }
    // ---- per sub-tile: input, layer 1 over the 180 halo pixels, hidden tile ----
    for (int sb = 0; sb < kDecSub; ++sb) {
      if (!prefetch || it == 0) bad |= load_input_tile(feat, W, H, Cin, K1, ty0[sb], tx0[sb], smem + kSmA0, tid, kDecThreads);
      fence_async_smem();
      tc_fence_before();
      if (!__syncthreads_and(ok)) { ok = false; break; }
      // rows 0..127 -> columns [0, Ch), rows 52..179 -> [128, 128 + Ch)
      if (tid == 0) {
        const uint32_t wb = acquire(gbase);
        if (ok) {
          const uint64_t bd = smem_desc(wb, Ch * 16, 128);
          for (int mt = 0; mt < 2; ++mt)
            mma_chain(tmem + mt * 128, smem_desc(a0 + mt * 52 * 16, kA0Pitch * 16, 128), bd, 2 * kA0Pitch, 2 * Ch, K1 >> 4,
                      idesc_h, false);
          mma_commit(bar_m);
          if (sb == kDecSub - 1) release(gbase);
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);
      ph_m ^= 1u;
      tc_fence_after();
      if (ok) {
        char* s_h1 = smem + kSmH1 + sb * kDecH1Bytes;
        for (int mt = 0; mt < 2; ++mt) {
          if (mt == 1 && q < 2) continue;               // rows 52..115 of the second product repeat the first
          const int r = mt * 52 + q * 32 + lane;
          const bool store = mt == 0 || r >= 128;
          const int hy = r / kHaloW, hx = r - hy * kHaloW;
          const int y = ty0[sb] + hy - 1, x = tx0[sb] + hx - 1;
          const bool inside = y >= 0 && y < H && x >= 0 && x < W;   // outside: the 3x3 convolution's zero padding
          for (int cc = hsel; cc < (Ch >> 5); cc += kColGroups) {
            uint32_t acc[32];
            tmem_ld32(trow + mt * 128 + cc * 32, acc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 w;
              bad |= relu_pack(acc, s_bias + cc * 32, j, w);
              if (store) *reinterpret_cast<uint4*>(s_h1 + ((cc * 4 + j) * kHaloPx + r) * 16) = inside ? w : make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (!__syncthreads_and(ok)) { ok = false; break; }
    }
    if (!ok) break;
    // ---- layer 2: nine taps, each weight block serves every sub-tile; columns [256 + 128 sb, .. + Ch) ----
    // While one lane issues them, the other warps fetch the next tile's input: layer 1 has finished
    // reading the input tile.
    if (warp != 0) {
      if (prefetch && it + 1 < n_my) {
        const int nt = ((int)blockIdx.x + (it + 1) * (int)gridDim.x) * kDecSub;
        bad |= load_input_tile(feat, W, H, Cin, K1, (nt / tiles_x) * kDecTileH, (nt % tiles_x) * kDecTileW, smem + kSmA0,
                               tid - 32, kDecThreads - 32);
      }
    } else if (tid == 0) {
      for (int tap = 0; tap < 9 && ok; ++tap) {
        const int g = gbase + 1 + tap;
        const uint32_t wb = acquire(g);
        if (!ok) break;
        const int shift = (tap / 3) * kHaloW + tap % 3;
        const uint64_t bd = smem_desc(wb, Ch * 16, 128);
        for (int sb = 0; sb < kDecSub; ++sb)
          mma_chain(tmem + 256 + sb * 128, smem_desc(h1 + sb * kDecH1Bytes + shift * 16, kHaloPx * 16, kHaloW * 16), bd,
                    2 * kHaloPx, 2 * Ch, Ch >> 4, idesc_h, tap != 0);
        release(g);
      }
      if (ok) mma_commit(bar_m);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);
    ph_m ^= 1u;
    tc_fence_after();
    const int m = q * 32 + lane;                       // this thread's output pixel of either sub-tile
    if (ok) {
      for (int sb = 0; sb < kDecSub; ++sb)
        for (int cc = hsel; cc < (Ch >> 5); cc += kColGroups) {
          uint32_t acc[32];
          tmem_ld32(trow + 256 + sb * 128 + cc * 32, acc);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            bad |= relu_pack(acc, s_bias + Ch + cc * 32, j, w);
            // the hidden tile of layer 3 reuses the halo tile: every MMA that read it has finished
            *reinterpret_cast<uint4*>(smem + kSmH1 + sb * kDecH1Bytes + ((cc * 4 + j) * 128 + m) * 16) = w;
          }
        }
    }
    fence_async_smem();
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 3 in chunks of <= 128 output columns; sub-tile sb accumulates in columns [128 sb, ..) ----
    float best[kDecSub];
    int arg[kDecSub];
#pragma unroll
    for (int sb = 0; sb < kDecSub; ++sb) { best[sb] = -3.0e38f; arg[sb] = 0; }
    for (int c = 0; c < out_chunks; ++c) {
      const int nc = min(128, n_pad - c * 128);
      if (tid == 0) {
        const int g = gbase + 10 + c;
        const uint32_t wb = acquire(g);
        if (ok) {
          const uint64_t bd = smem_desc(wb, nc * 16, 128);
          for (int sb = 0; sb < kDecSub; ++sb)
            mma_chain(tmem + sb * 128, smem_desc(h1 + sb * kDecH1Bytes, 128 * 16, 128), bd, 2 * 128, 2 * nc, Ch >> 4,
                      instr_desc(128, nc), false);
          mma_commit(bar_o);
          release(g);
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar_o, ph_o) && ok);
      ph_o ^= 1u;
      tc_fence_after();
      if (ok) {
#pragma unroll
        for (int sb = 0; sb < kDecSub; ++sb) {
          // decoded features: the first eight warps only (one staging tile each)
          for (int cc = hsel; cc < (nc >> 5) && (classify || hsel < 2); cc += classify ? kColGroups : 2) {
            uint32_t acc[32];
            tmem_ld32(trow + sb * 128 + cc * 32, acc);
            const int col0 = c * 128 + cc * 32;
            const float* b3 = s_bias + 2 * Ch + col0;
            if (classify) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const float v = __uint_as_float(acc[e]) + b3[e];
                if (col0 + e < n_out && v > best[sb]) { best[sb] = v; arg[sb] = col0 + e; }
              }
            } else {
              // 32 pixels x 32 columns of this warp go through a staging tile so that eight lanes write one pixel's
              // 128 contiguous bytes; the 16-byte unit u of pixel row l sits at unit u ^ (l & 7): both the row
              // writes and the transposed reads touch every bank once per eight lanes
              float* stg = reinterpret_cast<float*>(smem + kSmStage) + warp * kStageFloats;
              __syncwarp();
#pragma unroll
              for (int e = 0; e < 32; e += 4)
                *reinterpret_cast<float4*>(stg + lane * 32 + (((e >> 2) ^ (lane & 7)) << 2)) =
                    make_float4(__uint_as_float(acc[e]) + b3[e], __uint_as_float(acc[e + 1]) + b3[e + 1],
                                __uint_as_float(acc[e + 2]) + b3[e + 2], __uint_as_float(acc[e + 3]) + b3[e + 3]);
              __syncwarp();
              const int cq = (lane & 7) * 4;
#pragma unroll
              for (int rr = 0; rr < 32; rr += 4) {
                const int ml = rr + (lane >> 3), mm = q * 32 + ml;            // pixel of the tile this lane writes for
                const int oy = ty0[sb] + (mm >> 3), ox = tx0[sb] + (mm & 7);
                if (oy < H && ox < W) {
                  const float4 v = *reinterpret_cast<const float4*>(stg + ml * 32 + ((((cq >> 2)) ^ (ml & 7)) << 2));
                  float* dst = out + ((int64_t)oy * W + ox) * n_out + col0 + cq;
                  if ((n_out & 3) == 0) {
                    if (col0 + cq < n_out) *reinterpret_cast<float4*>(dst) = v;
                  } else {
                    if (col0 + cq < n_out) dst[0] = v.x;
                    if (col0 + cq + 1 < n_out) dst[1] = v.y;
                    if (col0 + cq + 2 < n_out) dst[2] = v.z;
                    if (col0 + cq + 3 < n_out) dst[3] = v.w;
                  }
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      if (!__syncthreads_and(ok)) { ok = false; break; }
    }
    if (!ok) break;
    if (classify) {
      // the column interleaves of a pixel meet here; the lower class index wins a tie
#pragma unroll
      for (int sb = 0; sb < kDecSub; ++sb) s_arg[(sb * kColGroups + hsel) * 128 + m] = make_float2(best[sb], __int_as_float(arg[sb]));
      __syncthreads();
      if (hsel == 0) {
#pragma unroll
        for (int sb = 0; sb < kDecSub; ++sb) {
          const int py = ty0[sb] + (m >> 3), px = tx0[sb] + (m & 7);
          float bv = best[sb];
          int a = arg[sb];
          for (int g = 1; g < kColGroups; ++g) {
            const float2 o = s_arg[(sb * kColGroups + g) * 128 + m];
            const int oa = __float_as_int(o.y);
            if (o.x > bv || (o.x == bv && oa < a)) { bv = o.x; a = oa; }
          }
          if (py < H && px < W) labels[(int64_t)py * W + px] = a;
        }
      }
      __syncthreads();
    }
  }

  if (!ok && tid == 0) {
    atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TIMEOUT);
    // copies requested but never waited for may still be in flight: give each a bounded chance to land
    // before the shared memory is released
    for (int j = landed; j < issued; ++j) mbar_wait(bar_full + 8 * (j % kDecRing), (uint32_t)((j / kDecRing) & 1));
  }
  if (bad) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 512);
}

// ------------------------------------------------------- text query of a full-width feature map ----
// logits [P x C] = feat [P x D] . text^T [D x C] as a register-tiled FP32 product on the CUDA cores: a block owns
// 128 pixels and walks the classes in tiles of CT; per step of 16 feature channels the two operand tiles are
// staged k-major in shared memory (next step's global loads in flight meanwhile) and each thread accumulates
// 4 pixels x CT/8 classes from 16-byte shared loads (the class values are a warp-wide broadcast).
// logit = (f . t_c) / max(|t_c|, 1e-12); the per-pixel normalisation of the reference is one positive factor for
// all classes and does not enter the comparison (an all-zero row gives label 0 either way).  The first maximum
// wins, like torch.argmax: threads hold ascending classes, class groups and class tiles are merged in ascending
// order, and only a strictly larger logit replaces the winner.
constexpr int kMaxClasses = 1024;
constexpr int kQM = 128, kQK = 16, kQPitchA = kQM + 4;
template <int CT>
__global__ void __launch_bounds__(256) k_classify_features(const float* __restrict__ feat, int64_t P, int D,
                                                           const float* __restrict__ text, int C,
                                                           long long* __restrict__ labels) {
  constexpr int TN = CT / 8, kPitchB = CT + 4;
  __shared__ __align__(16) float s_a[2][kQK][kQPitchA];
  __shared__ __align__(16) float s_b[2][kQK][kPitchB];
  __shared__ float s_inv[kMaxClasses];
  __shared__ float s_val[8][kQM];
  __shared__ int s_idx[8][kQM];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  for (int c = warp; c < C; c += 8) {
    float ss = 0.f;
    for (int k = lane; k < D; k += 32) { const float v = __ldg(text + (int64_t)c * D + k); ss = fmaf(v, v, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_inv[c] = 1.0f / fmaxf(sqrtf(ss), 1e-12f);
  }
  const int64_t p0 = (int64_t)blockIdx.x * kQM;
  const bool vec = (D & 3) == 0;
  const int lk = (t & 3) * 4;                 // this thread's 4 channels of a 16-channel step
  const int lrow = t >> 2;                    // pixel (two: +0, +64) or class row it loads
  const int steps = (D + kQK - 1) / kQK;
  // one 16-byte piece of a row, zero beyond the row's end or the matrix's
  auto fetch = [&](const float* base, int64_t row, int64_t rows, int k) -> float4 {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < rows) {
      const float* src = base + row * D + k;
      if (vec) { if (k < D) v = __ldg(reinterpret_cast<const float4*>(src)); }
      else {
        if (k < D) v.x = __ldg(src);
        if (k + 1 < D) v.y = __ldg(src + 1);
        if (k + 2 < D) v.z = __ldg(src + 2);
        if (k + 3 < D) v.w = __ldg(src + 3);
      }
    }
    return v;
  };
  auto put = [&](float (*dst)[kQPitchA], int col, const float4& v) {
    dst[lk][col] = v.x; dst[lk + 1][col] = v.y; dst[lk + 2][col] = v.z; dst[lk + 3][col] = v.w;
  };
  auto put_b = [&](float (*dst)[kPitchB], int col, const float4& v) {
    dst[lk][col] = v.x; dst[lk + 1][col] = v.y; dst[lk + 2][col] = v.z; dst[lk + 3][col] = v.w;
  };
  float run_val = -3.0e38f;                    // threads 0..127: the winner so far of pixel p0 + t
  int run_idx = 0;
  __syncthreads();
  for (int c0 = 0; c0 < C; c0 += CT) {
    float acc[4][TN];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    float4 ra0 = fetch(feat, p0 + lrow, P, lk), ra1 = fetch(feat, p0 + lrow + 64, P, lk);
    float4 rb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lrow < CT) rb = fetch(text, c0 + lrow, C, lk);
    put(s_a[0], lrow, ra0); put(s_a[0], lrow + 64, ra1);
    if (lrow < CT) put_b(s_b[0], lrow, rb);
    __syncthreads();
    for (int st = 0; st < steps; ++st) {
      const int cur = st & 1;
      if (st + 1 < steps) {
        const int k = (st + 1) * kQK + lk;
        ra0 = fetch(feat, p0 + lrow, P, k); ra1 = fetch(feat, p0 + lrow + 64, P, k);
        if (lrow < CT) rb = fetch(text, c0 + lrow, C, k);
      }
#pragma unroll
      for (int k = 0; k < kQK; ++k) {
        const float4 a = *reinterpret_cast<const float4*>(&s_a[cur][k][lane * 4]);
        float b[TN];
#pragma unroll
        for (int j = 0; j < TN; j += 4) {
          const float4 bv = *reinterpret_cast<const float4*>(&s_b[cur][k][warp * TN + j]);
          b[j] = bv.x; b[j + 1] = bv.y; b[j + 2] = bv.z; b[j + 3] = bv.w;
        }
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[0][j] = fmaf(a.x, b[j], acc[0][j]); acc[1][j] = fmaf(a.y, b[j], acc[1][j]);
          acc[2][j] = fmaf(a.z, b[j], acc[2][j]); acc[3][j] = fmaf(a.w, b[j], acc[3][j]);
        }
      }
      if (st + 1 < steps) {
        put(s_a[cur ^ 1], lrow, ra0); put(s_a[cur ^ 1], lrow + 64, ra1);
        if (lrow < CT) put_b(s_b[cur ^ 1], lrow, rb);
      }
      __syncthreads();
    }
    // this thread's best class per pixel, then the eight class groups of the tile in ascending order
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float bv = -3.0e38f;
      int bi = 0;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int c = c0 + warp * TN + j;
        if (c < C) {
          const float v = acc[i][j] * s_inv[c];
          if (v > bv) { bv = v; bi = c; }
        }
      }
      s_val[warp][lane * 4 + i] = bv;
      s_idx[warp][lane * 4 + i] = bi;
    }
    __syncthreads();
    if (t < kQM) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float v = s_val[g][t];
        if (v > run_val) { run_val = v; run_idx = s_idx[g][t]; }
      }
    }
    __syncthreads();
  }
  if (t < kQM && p0 + t < P) labels[p0 + t] = run_idx;
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int64_t mlpsp_decoder_packed_bytes(const mlpsp_decoder* dec, int32_t mode) {
  DecHeader h;
  if (!dec || (mode != 0 && mode != 1) || !dec_layout(dec, mode, &h)) return 0;
  // the folded text matrix and its bias are staged behind the image while packing
  return (int64_t)h.total_bytes + (mode == 1 ? 4ll * (dec->num_classes * (dec->hidden + 1)) + 256 : 0);
}

extern "C" int mlpsp_pack_decoder(const mlpsp_decoder* dec, int32_t mode, void* packed, int32_t* status, void* stream) {
  MLPSP_REQUIRE(dec && packed, MLPSP_E_ARG, "mlpsp_pack_decoder: null pointer");
  MLPSP_REQUIRE(mode == 0 || mode == 1, MLPSP_E_ARG, "mlpsp_pack_decoder: mode is 0 (decoded features) or 1 (text query)");
  MLPSP_REQUIRE(dec->W1 && dec->b1 && dec->W2 && dec->b2 && dec->W3 && dec->b3, MLPSP_E_ARG, "mlpsp_pack_decoder: weights missing");
  MLPSP_REQUIRE(mode == 0 || (dec->text && dec->num_classes > 0), MLPSP_E_ARG, "mlpsp_pack_decoder: a text query needs the text embeddings");
  DecHeader h;
  MLPSP_REQUIRE(dec_layout(dec, mode, &h), MLPSP_E_LIMIT,
                "mlpsp_pack_decoder: input width 1..128, hidden width 32, 64, 96 or 128, at most %d outputs or classes", kDecMaxOut);
  MLPSP_REQUIRE(dec->out_dim * 4 <= 160 * 1024, MLPSP_E_LIMIT, "mlpsp_pack_decoder: output width beyond 40960");
  cudaStream_t st = (cudaStream_t)stream;
  LaunchScope scope(kKMisc, 2, st);
  float* folded = nullptr;
  float* fb = nullptr;
  if (mode == 1) {
    folded = reinterpret_cast<float*>((char*)packed + h.total_bytes);
    fb = folded + (size_t)dec->num_classes * dec->hidden;
    static DeviceOnce fold_once;
    if (fold_once.first()) {
      MLPSP_CUDA_OK(cudaFuncSetAttribute(k_fold_text, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    }
    k_fold_text<<<dec->num_classes, 128, dec->out_dim * 4, st>>>(dec->text, dec->W3, dec->b3, dec->out_dim, dec->hidden, folded, fb);
  }
  k_pack_decoder<<<64, 256, 0, st>>>(h, dec->W1, dec->b1, dec->W2, dec->b2, dec->W3, dec->b3, folded, fb, (char*)packed, status);
  return cuda_check(cudaGetLastError(), "mlpsp_pack_decoder");
}

extern "C" int mlpsp_decode_features(const mlpsp_decoder* dec, int32_t mode, const void* packed, const float* feat,
                                     int32_t width, int32_t height, float* out, int64_t* labels, int32_t* status,
                                     void* stream) {
  MLPSP_REQUIRE(dec && packed && feat && status, MLPSP_E_ARG, "mlpsp_decode_features: null pointer");
  MLPSP_REQUIRE(width > 0 && height > 0, MLPSP_E_ARG, "mlpsp_decode_features: empty image");
  MLPSP_REQUIRE((mode == 0 && out) || (mode == 1 && labels), MLPSP_E_ARG,
                "mlpsp_decode_features: mode 0 writes out, mode 1 writes labels");
  DecHeader h;
  MLPSP_REQUIRE(dec_layout(dec, mode, &h), MLPSP_E_LIMIT, "mlpsp_decode_features: decoder sizes outside the kernel's limits");
  MLPSP_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 15) == 0 && (reinterpret_cast<uintptr_t>(feat) & 15) == 0 &&
                (mode == 1 || (reinterpret_cast<uintptr_t>(out) & 15) == 0), MLPSP_E_ARG,
                "mlpsp_decode_features: buffers must be 16-byte aligned");
  static DeviceOnce decode_once;
  if (decode_once.first()) {
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_decode_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles_x = (width + kDecTileW - 1) / kDecTileW, tiles_y = (height + kDecTileH - 1) / kDecTileH;
  const int num_tiles = tiles_x * tiles_y;
  cudaStream_t st = (cudaStream_t)stream;
  LaunchScope scope(kKMisc, 1, st);
  k_decode_tc<<<std::min((num_tiles + kDecSub - 1) / kDecSub, sms), kDecThreads, kDecSmem, st>>>((const char*)packed, feat, width, height, tiles_x, num_tiles,
                                                                     out, reinterpret_cast<long long*>(labels), status);
  return cuda_check(cudaGetLastError(), "mlpsp_decode_features");
}

extern "C" int mlpsp_classify_features(const float* feat, int64_t pixels, int32_t dim, const float* text,
                                       int32_t num_classes, int64_t* labels, void* stream) {
  MLPSP_REQUIRE(feat && text && labels, MLPSP_E_ARG, "mlpsp_classify_features: null pointer");
  MLPSP_REQUIRE(pixels >= 0 && dim > 0 && num_classes > 0, MLPSP_E_ARG, "mlpsp_classify_features: bad sizes");
  MLPSP_REQUIRE(num_classes <= kMaxClasses && pixels <= (int64_t)kQM * 0x7fffffff, MLPSP_E_LIMIT,
                "mlpsp_classify_features: at most %d classes", kMaxClasses);
  if (pixels == 0) return MLPSP_OK;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaStream_t st = (cudaStream_t)stream;
  LaunchScope scope(kKMisc, 1, st);
  long long* lab = reinterpret_cast<long long*>(labels);
  const int grid = (int)((pixels + kQM - 1) / kQM);
  if (num_classes <= 32) k_classify_features<32><<<grid, 256, 0, st>>>(feat, pixels, dim, text, num_classes, lab);
  else k_classify_features<64><<<grid, 256, 0, st>>>(feat, pixels, dim, text, num_classes, lab);
  return cuda_check(cudaGetLastError(), "mlpsp_classify_features");
}
