// Per-primitive MLP evaluator on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// What the reference does per (tile, primitive) with warp-level wmma on 64 rays
// (scannet/cuda/rgb_wmma.cuh:75-223) is done here per (primitive, 128 of its records):
//   * the primitive's fp16 weight image (pre-packed once per scene in the canonical K-major
//     core-matrix layout) arrives in shared memory by one TMA bulk copy (cp.async.bulk) that
//     signals an mbarrier;
//   * each of the 128 threads encodes one record (sin/cos of v6 * freq * att, rounded to fp16,
//     72 values padded to 80) straight into the A-operand tile in shared memory;
//   * layer 1 (128x80 . 80x32), layer 2 (128x32 . 32x32) and layer 3 (128x32 . 32x16, 4 columns
//     used) are tcgen05.mma.kind::f16 instructions issued by one thread, FP32 accumulators in
//     tensor memory; between layers every thread pulls its own accumulator row back with
//     tcgen05.ld, adds the FP32 bias, applies ReLU, rounds to fp16 and writes the next A tile;
//   * the epilogue applies sigmoid / softplus (and 1-exp(-sigma*decay)) and scatters one float4
//     per record to its compositing slot.
// Numerics follow the reference's tensor-core contract: operands and hidden activations rounded
// to binary16 (RN), FP32 accumulation from zero, FP32 bias added afterwards.
//
// Every wait on an mbarrier is bounded; when one gives up the CTA raises MLPSP_ST_TIMEOUT, waits
// (bounded) for its own bulk copy, frees its tensor memory and returns.
#include "frame.cuh"
#include "tc.cuh"

namespace mlpsp {

// ---- packed weight image (bytes, per primitive) for F = 6 and hidden width H = 32 or 64 ----
constexpr int kK1 = 80;                  // 72 encoded inputs padded to a multiple of 16
constexpr int kN3 = 16;                  // 4 outputs padded to the smallest N
constexpr int kRows = kRowsPerItem;      // 128 = MMA M
constexpr int kA1Bytes = 9 * kRows * 16;          // 18432: [9 k-chunks][128][8 halves], 72 encoded inputs

template <int H>
struct Net {
  static_assert(H == 32 || H == 64, "hidden width of the tensor-core evaluator");
  // W1: [10 k-chunks][H rows][8 halves]: chunks 0..7 of K in the order of enc_k(), an all-zero chunk, then
  // chunk 8 (see the last layer-1 MMA); W2: [H/8][H][8]; W3: [H/8][16][8] (rows 4..15 zero); b1[H] b2[H] b3[4] FP32
  static constexpr int kOffW1 = 0;
  static constexpr int kOffW2 = kOffW1 + (kK1 / 8) * H * 16;
  static constexpr int kOffW3 = kOffW2 + (H / 8) * H * 16;
  static constexpr int kOffBias = kOffW3 + (H / 8) * kN3 * 16;
  static constexpr int kWeightBytes = kOffBias + 4 * (H + H + 4);   // 8,464 (H = 32) / 21,008 (H = 64), multiples of 16
  static constexpr int kA2Bytes = (H / 8) * kRows * 16;             // hidden tile, reuses the layer-1 A tile
  static_assert(kA2Bytes <= kA1Bytes && kWeightBytes % 16 == 0, "tile aliasing / bulk-copy granularity");
  static constexpr int kSmemBytes = kWeightBytes + kA1Bytes + 64;
  static constexpr int kTmemCols = 2 * H;   // D1 [0,H)  D2 [H,2H)  D3 reuses [0,16)
  // resident CTAs per SM: H = 32: shared memory (28 KB), registers (64) and tensor memory (64 columns) all give 8;
  // H = 64: tensor memory (128 columns) gives 4
  static constexpr int kCtas = H == 32 ? 8 : 4;
};

// Position of an encoded input inside the K dimension of layer 1.  The reference orders K as
// [sin(c,f) for c, f][cos(c,f) for c, f] (np_tile_kernels.cu:329-343); a dot product does not care, so
// the A tile and the packed W1 rows both use an order in which the six (sin, cos) pairs of one input
// coordinate are contiguous and two coordinates fill exactly three 16-byte chunks:
//   k' = 12 c + 4 (f / 2) + 2 is_cos + (f % 2).
__host__ __device__ constexpr int enc_k(int c, int f, int is_cos) { return 12 * c + 4 * (f >> 1) + 2 * is_cos + (f & 1); }
__host__ __device__ constexpr int enc_k_of_reference(int k) {
  return k >= 72 ? k : enc_k((k % 36) / 6, (k % 36) % 6, k / 36);
}

// hidden layer epilogue: +bias, ReLU, fp16 (RN), write this thread's row of the next A tile.
// Returns true when an activation rounded to +inf in binary16.  The FP32 sums themselves are always
// finite: operands are finite fp16 values, so |sum| <= 80 * 65504^2 (rgb_wmma.cuh:179-181 checks for a
// non-finite or fp16-overflowing activation per element).
template <bool KEEP, bool BF16>
__device__ __forceinline__ bool hidden_to_smem(const uint32_t (&acc)[32], const float* bias, char* a2, int row,
                                               uint32_t& relu_mask) {
  // running maximum of the packed activations (they are >= 0 after the ReLU, so for both formats the bit
  // patterns order like the values and one unsigned 16-bit-lane maximum serves either)
  uint32_t top = 0u;
  relu_mask = 0u;
#pragma unroll
  for (int kc = 0; kc < 4; ++kc) {
    const float4 b0 = *reinterpret_cast<const float4*>(bias + kc * 8);
    const float4 b1 = *reinterpret_cast<const float4*>(bias + kc * 8 + 4);
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = kc * 8 + q * 2;
      const float v0 = __uint_as_float(acc[j]) + bb[q * 2], v1 = __uint_as_float(acc[j + 1]) + bb[q * 2 + 1];
      if (KEEP) {
        relu_mask |= (v0 > 0.f ? 1u : 0u) << j;
        relu_mask |= (v1 > 0.f ? 1u : 0u) << (j + 1);
      }
      w[q] = pack_h2_relu<BF16>(v0, v1);
      top = __vmaxu2(top, w[q]);
    }
    *reinterpret_cast<uint4*>(a2 + kc * (kRows * 16) + row * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // +inf (or the canonical NaN a non-finite sum converts to) in either lane
  const uint32_t inf16 = BF16 ? 0x7f80u : 0x7c00u;
  return (top & 0xffffu) >= inf16 || (top >> 16) >= inf16;
}

// Encode one record into this thread's row of the layer-1 A tile (K order of enc_k()).  mult[f] is
// freq[f] * att[f].  LADDER: every band is exactly twice the one before, so the phases are exact
// doublings of the first and sin / cos of the higher bands follow from the double-angle identities
// (2 special-function evaluations per coordinate instead of 12).  Returns true for a non-finite input.
template <bool LADDER, bool BF16>
__device__ __forceinline__ bool encode_row(const RecIn& r, const float (&mult)[6], char* row_ptr) {
  const float v6[6] = {r.rdx, r.rdy, r.rdz, r.dx, r.dy, r.dz};
  bool bad = false;
#pragma unroll
  for (int cp = 0; cp < 3; ++cp) {
    uint32_t w[12];
#pragma unroll
    for (int d = 0; d < 2; ++d) {
      const float v = v6[cp * 2 + d];
      bad |= !(fabsf(v) < 1.0e30f);   // a finite input gives finite phases (freq * att <= 101)
      float sn[6], cs[6];
      if (LADDER) {
        __sincosf(v * mult[0], &sn[0], &cs[0]);
#pragma unroll
        for (int f = 1; f < 6; ++f) {
          const float t = sn[f - 1] + sn[f - 1];
          sn[f] = t * cs[f - 1];
          cs[f] = fmaf(-t, sn[f - 1], 1.0f);
        }
      } else {
#pragma unroll
        for (int f = 0; f < 6; ++f) __sincosf(v * mult[f], &sn[f], &cs[f]);
      }
#pragma unroll
      for (int g = 0; g < 3; ++g) {
        w[d * 6 + g * 2] = pack_h2<BF16>(sn[2 * g], sn[2 * g + 1]);
        w[d * 6 + g * 2 + 1] = pack_h2<BF16>(cs[2 * g], cs[2 * g + 1]);
      }
    }
#pragma unroll
    for (int q = 0; q < 3; ++q)
      *reinterpret_cast<uint4*>(row_ptr + (cp * 3 + q) * (kRows * 16)) =
          make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
  }
  return bad;
}

// One work item = (primitive, first record, rows <= 128).  Items are dealt to CTAs round-robin
// (item = blockIdx.x + k * gridDim.x): all items cost about the same, and a fixed deal lets a CTA
// fetch the next item's descriptor, its record and -- as soon as the MMAs that read them have
// finished -- the next primitive's W1 and W2 blocks while the current item is still being evaluated,
// so the only global-memory latency left on an item's critical path is the 1.3 KB copy of W3 + biases.
template <bool KEEP, bool BF16, int H>
__global__ void __launch_bounds__(kRows, KEEP ? 6 : Net<H>::kCtas) k_mlp_tc(
    const char* __restrict__ w16, const float* __restrict__ freq, const float* __restrict__ att,
    const RecIn* __restrict__ rec_in, const int4* __restrict__ work,
    const int32_t* __restrict__ counters, float4* __restrict__ rec_out, float4* __restrict__ rec_ext, int out_mode,
    int32_t* __restrict__ status) {
  using N = Net<H>;
  static_assert(!KEEP || H == 32, "the record export keeps 32-bit ReLU masks");
  extern __shared__ __align__(128) char smem[];
  char* s_w = smem;
  char* s_a1 = smem + N::kWeightBytes;
  char* s_a2 = s_a1;                         // written only after the layer-1 MMAs have finished reading s_a1
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_a1 + kA1Bytes);   // [0] weights, [1] mma
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 2);        // [0] tmem base
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = counters[kCtrWork];
  int item = blockIdx.x;
  if (item >= G) return;                     // more CTAs than work: leave before touching tensor memory
  const uint32_t bar_w = smem_u32(&s_bar[0]), bar_m = smem_u32(&s_bar[1]);
  const uint32_t a1 = smem_u32(s_a1), a2 = smem_u32(s_a2), wb = smem_u32(s_w);
  int4 wk = __ldg(work + item);
  if (tid == 0) {
    mbar_init(bar_w, 1);
    mbar_init(bar_m, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
    // the first item's whole weight image
    mbar_expect_tx(bar_w, N::kWeightBytes);
    bulk_g2s(wb, w16 + (size_t)wk.x * N::kWeightBytes, N::kWeightBytes, bar_w);
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_misc[0]), N::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes
  // phase multipliers freq[f] * att[f]; when every band is exactly twice the one before (equal
  // attenuation: FourierFeatureEncoding's bands, cumodel.py:163) the encoder takes the double-angle route
  float mult[6];
  bool ladder = true;
#pragma unroll
  for (int f = 0; f < 6; ++f) mult[f] = __ldg(freq + f) * __ldg(att + f);
#pragma unroll
  for (int f = 1; f < 6; ++f) ladder = ladder && mult[f] == 2.0f * mult[f - 1];
  const float* s_bias = reinterpret_cast<const float*>(s_w + N::kOffBias);
  uint32_t ph_w = 0, ph_m = 0;
  bool ok = true, bad = false, copy_pending = true;
  uint32_t relu1 = 0u, relu2 = 0u;
  RecIn r;
  r.rdx = r.rdy = r.rdz = r.dx = r.dy = r.dz = 0.f; r.decay = 0.f; r.slot = 0u;
  if (tid < wk.z) r = rec_in[wk.y + tid];

  for (;;) {
    const int nrows = wk.z;
    const bool valid = tid < nrows;
    // MMA rows are independent and rows past the end of the primitive's records are never stored, so a
    // warp whose 32 rows are all past the end skips the encoding and the epilogues (its rows of the
    // operand tiles keep whatever they held) and only takes part in the barriers
    const bool warp_live = warp * 32 < nrows;
    const int next = item + (int)gridDim.x;
    const bool has_next = next < G;
    int4 wk_next = make_int4(0, 0, 0, 0);
    const float decay = r.decay;
    const uint32_t slot = r.slot;
    // ---- encode this thread's record into the layer-1 A tile ----
    if (warp_live) {
      // rows past the end inside a live warp hold the zero record; their results are never stored
      const bool nonfinite = ladder ? encode_row<true, BF16>(r, mult, s_a1 + tid * 16)
                                    : encode_row<false, BF16>(r, mult, s_a1 + tid * 16);
      bad |= nonfinite;
    }
    fence_async_smem();
    {
      const bool landed = mbar_wait(bar_w, ph_w);   // weights landed (every thread reads the biases later)
      if (landed) { ph_w ^= 1u; copy_pending = false; }
      ok = ok && landed;
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 1: D1[128x32] = A1[128x72] . W1^T ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        mma_f16(tmem, smem_desc(a1 + ks * 2 * (kRows * 16), kRows * 16, 128),
                smem_desc(wb + N::kOffW1 + ks * 2 * (H * 16), H * 16, 128), instr_desc(kRows, H, BF16), ks > 0);
      // K = 64..79: the weight image holds a zero chunk and then chunk 8; the A operand pairs them with
      // chunk 7 (any finite values: they meet zeros) and chunk 8, so no padded A chunk is stored
      mma_f16(tmem, smem_desc(a1 + 7 * (kRows * 16), kRows * 16, 128),
              smem_desc(wb + N::kOffW1 + 8 * (H * 16), H * 16, 128), instr_desc(kRows, H, BF16), 1u);
      mma_commit(bar_m);
    }
    // the next item's descriptor and record are requested behind the proxy fence (which would otherwise
    // wait for them); their latency hides under the layers of this item
    if (has_next) wk_next = __ldg(work + next);
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
    ph_m ^= 1u;
    tc_fence_after();
    r.rdx = r.rdy = r.rdz = r.dx = r.dy = r.dz = 0.f; r.decay = 0.f; r.slot = 0u;
    if (tid < wk_next.z) r = rec_in[wk_next.y + tid];
    if (tid == 0 && has_next && ok) {
      // W1 is no longer read: start the next primitive's image with its W1 block
      mbar_expect_tx(bar_w, N::kWeightBytes);
      bulk_g2s(wb + N::kOffW1, w16 + (size_t)wk_next.x * N::kWeightBytes + N::kOffW1, N::kOffW2 - N::kOffW1, bar_w);
    }
    if (has_next && ok) copy_pending = true;
    if (ok && warp_live) {
#pragma unroll
      for (int part = 0; part < H / 32; ++part) {       // 32 accumulator columns = 4 K-chunks of the hidden tile at a time
        uint32_t acc[32];
        tmem_ld32(trow + part * 32, acc);
        bad |= hidden_to_smem<KEEP, BF16>(acc, s_bias + part * 32, s_a2 + part * 4 * (kRows * 16), tid, relu1) && valid;
      }
    }
    fence_async_smem();
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 2: D2[128x32] = H1[128x32] . W2^T ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < H / 16; ++ks)
        mma_f16(tmem + H, smem_desc(a2 + ks * 2 * (kRows * 16), kRows * 16, 128),
                smem_desc(wb + N::kOffW2 + ks * 2 * (H * 16), H * 16, 128), instr_desc(kRows, H, BF16), ks > 0);
      mma_commit(bar_m);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
    ph_m ^= 1u;
    tc_fence_after();
    if (tid == 0 && has_next && ok)
      bulk_g2s(wb + N::kOffW2, w16 + (size_t)wk_next.x * N::kWeightBytes + N::kOffW2, N::kOffW3 - N::kOffW2, bar_w);
    if (ok && warp_live) {                              // layer-2 MMAs have finished reading s_a2
#pragma unroll
      for (int part = 0; part < H / 32; ++part) {
        uint32_t acc[32];
        tmem_ld32(trow + H + part * 32, acc);
        bad |= hidden_to_smem<KEEP, BF16>(acc, s_bias + H + part * 32, s_a2 + part * 4 * (kRows * 16), tid, relu2) && valid;
      }
    }
    fence_async_smem();
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 3: D3[128x16] = H2[128x32] . W3^T (rows 4..15 of W3 are zero) ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < H / 16; ++ks)
        mma_f16(tmem, smem_desc(a2 + ks * 2 * (kRows * 16), kRows * 16, 128),
                smem_desc(wb + N::kOffW3 + ks * 2 * (kN3 * 16), kN3 * 16, 128), instr_desc(kRows, kN3, BF16), ks > 0);
      mma_commit(bar_m);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
    ph_m ^= 1u;
    tc_fence_after();
    if (ok && warp_live) {
      uint32_t o[4];
      tmem_ld4(trow, o);
      if (valid) {
        const float o0 = __uint_as_float(o[0]) + s_bias[2 * H + 0], o1 = __uint_as_float(o[1]) + s_bias[2 * H + 1];
        const float o2 = __uint_as_float(o[2]) + s_bias[2 * H + 2], o3 = __uint_as_float(o[3]) + s_bias[2 * H + 3];
        const float sigma_raw = softplus_fast(o3);
        float4 out;
        out.x = sigmoid_fast(o0); out.y = sigmoid_fast(o1); out.z = sigmoid_fast(o2);
        out.w = (out_mode == kOutAlpha) ? (1.f - __expf(-(sigma_raw * decay))) : sigma_raw;
        rec_out[slot] = out;
        if (KEEP) rec_ext[slot] = make_float4(sigma_raw, o3, __uint_as_float(relu1), __uint_as_float(relu2));
      }
    }
    tc_fence_before();
    // every thread is past its reads of the biases, W3 and the operand tiles of this item
    if (!__syncthreads_and(ok)) { ok = false; break; }
    if (!has_next) break;
    if (tid == 0)
      bulk_g2s(wb + N::kOffW3, w16 + (size_t)wk_next.x * N::kWeightBytes + N::kOffW3, N::kWeightBytes - N::kOffW3, bar_w);
    item = next;
    wk = wk_next;
  }

  if (!ok) {
    if (tid == 0) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TIMEOUT);
    // our own bulk copies may still be in flight: give them a bounded chance to land before the CTA's
    // shared memory is released (an image whose last block was never requested cannot complete; the
    // wait then simply runs out)
    if (copy_pending) mbar_wait(bar_w, ph_w);
  }
  if (bad) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, N::kTmemCols);
}

// ------------------------------------------------------------------------------ packing ----
template <bool BF16>
__device__ __forceinline__ uint16_t to_lp(float x, bool& bad) {
  if (BF16) {
    const __nv_bfloat16 v = __float2bfloat16_rn(x);
    bad |= __hisinf(v) || __hisnan(v);
    return *reinterpret_cast<const uint16_t*>(&v);
  }
  const __half v = __float2half_rn(x);
  bad |= __hisinf(v) || __hisnan(v);
  return *reinterpret_cast<const uint16_t*>(&v);
}

template <bool BF16, int H>
__global__ void k_pack_weights(const float* __restrict__ W1, const float* __restrict__ b1, const float* __restrict__ W2,
                               const float* __restrict__ b2, const float* __restrict__ W3, const float* __restrict__ b3,
                               int n, char* __restrict__ out, int32_t* __restrict__ status) {
  const int p = blockIdx.x;
  if (p >= n) return;
  using N = Net<H>;
  char* dst = out + (size_t)p * N::kWeightBytes;
  uint16_t* w1 = reinterpret_cast<uint16_t*>(dst + N::kOffW1);
  uint16_t* w2 = reinterpret_cast<uint16_t*>(dst + N::kOffW2);
  uint16_t* w3 = reinterpret_cast<uint16_t*>(dst + N::kOffW3);
  float* bias = reinterpret_cast<float*>(dst + N::kOffBias);
  bool bad = false;
  for (int i = threadIdx.x; i < H * kK1; i += blockDim.x) {
    const int h = i / kK1, k = i % kK1;
    const uint16_t v = to_lp<BF16>(k < 72 ? W1[(size_t)p * H * 72 + h * 72 + k] : 0.f, bad);
    const int kk = enc_k_of_reference(k);
    const int chunk = (kk >> 3) == 8 ? 9 : ((kk >> 3) == 9 ? 8 : (kk >> 3));   // zero chunk before the last real one
    w1[chunk * (H * 8) + h * 8 + (kk & 7)] = v;
  }
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) {
    const int h = i / H, k = i % H;
    const uint16_t v = to_lp<BF16>(W2[(size_t)p * H * H + i], bad);
    w2[(k >> 3) * (H * 8) + h * 8 + (k & 7)] = v;
  }
  for (int i = threadIdx.x; i < kN3 * H; i += blockDim.x) {
    const int h = i / H, k = i % H;
    const uint16_t v = to_lp<BF16>(h < 4 ? W3[(size_t)p * 4 * H + h * H + k] : 0.f, bad);
    w3[(k >> 3) * (kN3 * 8) + h * 8 + (k & 7)] = v;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    bias[i] = b1[(size_t)p * H + i];
    bias[H + i] = b2[(size_t)p * H + i];
    bad |= !isfinite(bias[i]) || !isfinite(bias[H + i]);
  }
  if (threadIdx.x < 4) { bias[2 * H + threadIdx.x] = b3[(size_t)p * 4 + threadIdx.x]; bad |= !isfinite(bias[2 * H + threadIdx.x]); }
  if (bad && status) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
}

template <int H>
static int launch_tc(const mlpsp_scene* sc, const char* image, const RecIn* rec_in, const int4* work,
                     const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                     cudaStream_t st, bool bf16, int grid_cap) {
  using N = Net<H>;
  static bool attr_set = false;
  if (!attr_set) {
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<false, false, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, N::kSmemBytes));
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<false, true, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, N::kSmemBytes));
    if (H == 32) {
      MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<true, false, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, Net<32>::kSmemBytes));
      MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<true, true, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, Net<32>::kSmemBytes));
    }
    attr_set = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms * (rec_ext ? 6 : N::kCtas);   // the record-export variant keeps two more words per row
  if (grid_cap > 0) grid = std::min(grid, grid_cap);
  LaunchScope scope(kKMlp, 1, st);
  if (rec_ext) {
    MLPSP_REQUIRE(H == 32, MLPSP_E_LIMIT, "record export needs hidden width 32 (32-bit ReLU masks)");
    if (bf16) k_mlp_tc<true, true, 32><<<grid, kRows, Net<32>::kSmemBytes, st>>>(image, sc->freq, sc->att, rec_in, work, counters,
                                                                               rec_out, rec_ext, out_mode, status);
    else k_mlp_tc<true, false, 32><<<grid, kRows, Net<32>::kSmemBytes, st>>>(image, sc->freq, sc->att, rec_in, work, counters,
                                                                            rec_out, rec_ext, out_mode, status);
  } else {
    if (bf16) k_mlp_tc<false, true, H><<<grid, kRows, N::kSmemBytes, st>>>(image, sc->freq, sc->att, rec_in, work, counters,
                                                                          rec_out, rec_ext, out_mode, status);
    else k_mlp_tc<false, false, H><<<grid, kRows, N::kSmemBytes, st>>>(image, sc->freq, sc->att, rec_in, work, counters,
                                                                       rec_out, rec_ext, out_mode, status);
  }
  return cuda_check(cudaGetLastError(), "mlp_f16");
}

int launch_mlp_f16(const mlpsp_scene* sc, const RecIn* rec_in, const int32_t* prim_off, const int4* work,
                   const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                   cudaStream_t st, bool bf16, int grid_cap) {
  MLPSP_REQUIRE((sc->hidden == 32 || sc->hidden == 64) && sc->num_freq == 6, MLPSP_E_LIMIT,
                "the tensor-core evaluator is built for 72->H->H->4 networks with H = 32 or 64 (6 frequencies)");
  const char* image = (const char*)(bf16 ? sc->wbf16 : sc->w16);
  MLPSP_REQUIRE(image && sc->freq && sc->att, MLPSP_E_ARG, "%s evaluator needs the packed weight image",
                bf16 ? "bf16" : "fp16");
  (void)prim_off;
  if (sc->hidden == 64)
    return launch_tc<64>(sc, image, rec_in, work, counters, rec_out, rec_ext, out_mode, status, st, bf16, grid_cap);
  return launch_tc<32>(sc, image, rec_in, work, counters, rec_out, rec_ext, out_mode, status, st, bf16, grid_cap);
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int64_t mlpsp_packed_weight_bytes(int32_t hidden, int32_t num_freq) {
  if (num_freq != 6) return 0;
  return hidden == 32 ? Net<32>::kWeightBytes : (hidden == 64 ? Net<64>::kWeightBytes : 0);
}

static int pack_weights(const mlpsp_scene* sc, void* out, int32_t* status, void* stream, bool bf16, const char* who) {
  MLPSP_REQUIRE(sc && out, MLPSP_E_ARG, "%s: null pointer", who);
  MLPSP_REQUIRE((sc->hidden == 32 || sc->hidden == 64) && sc->num_freq == 6, MLPSP_E_LIMIT,
                "%s: only 72->H->H->4 networks with H = 32 or 64 have a packed image", who);
  MLPSP_REQUIRE(sc->W1 && sc->b1 && sc->W2 && sc->b2 && sc->W3 && sc->b3, MLPSP_E_ARG, "%s: FP32 weights missing", who);
  if (sc->n == 0) return MLPSP_OK;
  cudaStream_t st = (cudaStream_t)stream;
  LaunchScope scope(kKMisc, 1, st);
#define MLPSP_PACK(BF, HH)                                                                                         \
  k_pack_weights<BF, HH><<<sc->n, 128, 0, st>>>(sc->W1, sc->b1, sc->W2, sc->b2, sc->W3, sc->b3, sc->n, (char*)out, status)
  if (sc->hidden == 64) { if (bf16) MLPSP_PACK(true, 64); else MLPSP_PACK(false, 64); }
  else { if (bf16) MLPSP_PACK(true, 32); else MLPSP_PACK(false, 32); }
#undef MLPSP_PACK
  return cuda_check(cudaGetLastError(), who);
}

extern "C" int mlpsp_pack_weights_f16(const mlpsp_scene* sc, void* w16_out, int32_t* status, void* stream) {
  return pack_weights(sc, w16_out, status, stream, false, "mlpsp_pack_weights_f16");
}

extern "C" int mlpsp_pack_weights_bf16(const mlpsp_scene* sc, void* wbf16_out, int32_t* status, void* stream) {
  return pack_weights(sc, wbf16_out, status, stream, true, "mlpsp_pack_weights_bf16");
}
