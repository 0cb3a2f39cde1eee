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

namespace mlpsp {

// ---- packed weight image (bytes, per primitive) for H = 32, F = 6 ----
constexpr int kK1 = 80;                  // 72 encoded inputs padded to a multiple of 16
constexpr int kH = 32;
constexpr int kN3 = 16;                  // 4 outputs padded to the smallest N
constexpr int kOffW1 = 0;                // [10 k-chunks][32 rows][8 halves]
constexpr int kOffW2 = kOffW1 + (kK1 / 8) * kH * 16;   // 5120: [4][32][8]
constexpr int kOffW3 = kOffW2 + (kH / 8) * kH * 16;    // 7168: [4][16][8]
constexpr int kOffBias = kOffW3 + (kH / 8) * kN3 * 16; // 8192: b1[32] b2[32] b3[4] fp32
constexpr int kWeightBytes = kOffBias + 4 * (kH + kH + 4);  // 8464, a multiple of 16

constexpr int kRows = kRowsPerItem;      // 128 = MMA M
constexpr int kA1Bytes = (kK1 / 8) * kRows * 16;  // 20480: [10][128][8 halves]
constexpr int kA2Bytes = (kH / 8) * kRows * 16;   // 8192:  [4][128][8 halves]
constexpr int kSmemBytes = kWeightBytes + kA1Bytes + 64;   // the hidden-activation tile reuses the layer-1 A tile
constexpr int kTmemCols = 64;            // D1 [0,32)  D2 [32,64)  D3 reuses [0,16)
constexpr int kSpinLimit = 1 << 20;

// -------------------------------------------------------------------------- PTX helpers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait: false when the phase did not complete within kSpinLimit polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try(bar, parity)) return true;
    if (i > 32) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// shared-memory matrix descriptor: K-major, no swizzle.  lbo = bytes between the two 8-element
// K chunks of one MMA, sbo = bytes between consecutive groups of 8 rows.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
         (1ull << 46);
}
// instruction descriptor: D = F32, A = B = F16, both K-major, dense
__host__ __device__ constexpr uint32_t instr_desc(int M, int N) {
  return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// hidden layer epilogue: +bias, ReLU, fp16, write this thread's row of the next A tile.
// Returns the largest |pre-activation| as an unsigned bit pattern (NaN and inf compare above every
// finite value), so the caller needs one comparison per layer to detect a non-finite sum or one that
// rounds to +inf in binary16 (rgb_wmma.cuh:179-181 checks the same two conditions per element).
template <bool KEEP>
__device__ __forceinline__ uint32_t hidden_to_smem(const uint32_t (&acc)[32], const float* bias, char* a2, int row,
                                                   uint32_t& relu_mask) {
  uint32_t worst = 0u;
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
      worst = max(worst, max(__float_as_uint(v0) & 0x7fffffffu, __float_as_uint(v1) & 0x7fffffffu));
      if (KEEP) {
        relu_mask |= (v0 > 0.f ? 1u : 0u) << j;
        relu_mask |= (v1 > 0.f ? 1u : 0u) << (j + 1);
      }
      w[q] = pack_h2(fmaxf(v0, 0.f), fmaxf(v1, 0.f));
    }
    *reinterpret_cast<uint4*>(a2 + kc * (kRows * 16) + row * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return worst;
}

constexpr uint32_t kHalfOverflowBits = 0x477ff000u;   // 65520.0f: the smallest magnitude that rounds to inf in binary16

template <bool KEEP>
__global__ void __launch_bounds__(kRows) k_mlp_tc(
    const char* __restrict__ w16, const float* __restrict__ freq, const float* __restrict__ att,
    const RecIn* __restrict__ rec_in, const int32_t* __restrict__ prim_off, const int2* __restrict__ work,
    int32_t* __restrict__ counters, float4* __restrict__ rec_out, float4* __restrict__ rec_ext, int out_mode,
    int32_t* __restrict__ status) {
  extern __shared__ __align__(128) char smem[];
  char* s_w = smem;
  char* s_a1 = smem + kWeightBytes;          // 8464 is a multiple of 16
  char* s_a2 = s_a1;                         // written only after the layer-1 MMAs have finished reading s_a1
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_a1 + kA1Bytes);   // [0] weights, [1] mma
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 2);        // [0] tmem base, [1] work item
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int G = counters[kCtrWork];
  if ((int)blockIdx.x >= G) return;          // more CTAs than work: leave before touching tensor memory
  const uint32_t bar_w = smem_u32(&s_bar[0]), bar_m = smem_u32(&s_bar[1]);
  if (tid == 0) {
    mbar_init(bar_w, 1);
    mbar_init(bar_m, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_misc[0]), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes
  float fr[6], at[6];
#pragma unroll
  for (int f = 0; f < 6; ++f) { fr[f] = __ldg(freq + f); at[f] = __ldg(att + f); }
  const uint32_t a1 = smem_u32(s_a1), a2 = smem_u32(s_a2), wb = smem_u32(s_w);
  const float* s_bias = reinterpret_cast<const float*>(s_w + kOffBias);
  uint32_t ph_w = 0, ph_m = 0;
  bool ok = true, bad = false, copy_pending = false;
  uint32_t relu1 = 0u, relu2 = 0u;

  for (;;) {
    if (tid == 0) s_misc[1] = (uint32_t)atomicAdd(counters + kCtrWorkNext, 1);
    __syncthreads();                          // also: previous item's reads of s_w / s_a* are done
    const int item = (int)s_misc[1];
    if (item >= G) break;
    const int2 wk = work[item];
    const int p = wk.x;
    const int pbase = prim_off[p];
    const int nrows = min(kRows, prim_off[p + 1] - pbase - wk.y);
    if (tid == 0) {
      mbar_expect_tx(bar_w, kWeightBytes);
      bulk_g2s(wb, w16 + (size_t)p * kWeightBytes, kWeightBytes, bar_w);
    }
    copy_pending = true;
    // ---- encode this thread's record into the layer-1 A tile ----
    const bool valid = tid < nrows;
    RecIn r;
    r.rdx = r.rdy = r.rdz = r.dx = r.dy = r.dz = 0.f; r.decay = 0.f; r.slot = 0u;
    if (valid) r = rec_in[pbase + wk.y + tid];
    {
      const float v6[6] = {r.rdx, r.rdy, r.rdz, r.dx, r.dy, r.dz};
      // rows past the end of the primitive's records encode the zero vector; their results are never stored
      float sn[36], cs[36];
#pragma unroll
      for (int c = 0; c < 6; ++c) {
        bad |= valid && !(fabsf(v6[c]) < 1.0e30f);   // a finite input gives finite phases (freq * att <= 101)
#pragma unroll
        for (int f = 0; f < 6; ++f) {
          const float ph = v6[c] * fr[f] * at[f];
          __sincosf(ph, &sn[c * 6 + f], &cs[c * 6 + f]);
        }
      }
      // k index: 0..35 sin block, 36..71 cos block, 72..79 zero (np_tile_kernels.cu:329-343)
#pragma unroll
      for (int kc = 0; kc < 10; ++kc) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j0 = kc * 8 + q * 2, j1 = j0 + 1;
          const float e0 = j0 < 36 ? sn[j0] : (j0 < 72 ? cs[j0 - 36] : 0.f);
          const float e1 = j1 < 36 ? sn[j1] : (j1 < 72 ? cs[j1 - 36] : 0.f);
          w[q] = pack_h2(e0, e1);
        }
        *reinterpret_cast<uint4*>(s_a1 + kc * (kRows * 16) + tid * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    fence_async_smem();
    {
      const bool landed = mbar_wait(bar_w, ph_w);   // weights landed (every thread reads the biases later)
      if (landed) { ph_w ^= 1u; copy_pending = false; }
      ok = ok && landed;
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 1: D1[128x32] = A1[128x80] . W1^T ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kK1 / 16; ++ks)
        mma_f16(tmem, smem_desc(a1 + ks * 2 * (kRows * 16), kRows * 16, 128),
                smem_desc(wb + kOffW1 + ks * 2 * (kH * 16), kH * 16, 128), instr_desc(kRows, kH), ks > 0);
      mma_commit(bar_m);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
    ph_m ^= 1u;
    tc_fence_after();
    {
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(trow, acc);
        bad |= valid && hidden_to_smem<KEEP>(acc, s_bias, s_a2, tid, relu1) >= kHalfOverflowBits;
      }
    }
    fence_async_smem();
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 2: D2[128x32] = H1[128x32] . W2^T ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kH / 16; ++ks)
        mma_f16(tmem + 32, smem_desc(a2 + ks * 2 * (kRows * 16), kRows * 16, 128),
                smem_desc(wb + kOffW2 + ks * 2 * (kH * 16), kH * 16, 128), instr_desc(kRows, kH), ks > 0);
      mma_commit(bar_m);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
    ph_m ^= 1u;
    tc_fence_after();
    {
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(trow + 32, acc);
        bad |= valid && hidden_to_smem<KEEP>(acc, s_bias + kH, s_a2, tid, relu2) >= kHalfOverflowBits;   // layer-2 MMAs have finished reading s_a2
      }
    }
    fence_async_smem();
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // ---- layer 3: D3[128x16] = H2[128x32] . W3^T (rows 4..15 of W3 are zero) ----
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kH / 16; ++ks)
        mma_f16(tmem, smem_desc(a2 + ks * 2 * (kRows * 16), kRows * 16, 128),
                smem_desc(wb + kOffW3 + ks * 2 * (kN3 * 16), kN3 * 16, 128), instr_desc(kRows, kN3), ks > 0);
      mma_commit(bar_m);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph_m) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
    ph_m ^= 1u;
    tc_fence_after();
    if (ok) {
      uint32_t o[4];
      tmem_ld4(trow, o);
      if (valid) {
        const float o0 = __uint_as_float(o[0]) + s_bias[2 * kH + 0], o1 = __uint_as_float(o[1]) + s_bias[2 * kH + 1];
        const float o2 = __uint_as_float(o[2]) + s_bias[2 * kH + 2], o3 = __uint_as_float(o[3]) + s_bias[2 * kH + 3];
        bad |= !(fabsf(o0) < 3.0e38f) || !(fabsf(o1) < 3.0e38f) || !(fabsf(o2) < 3.0e38f) || !(fabsf(o3) < 3.0e38f);
        const float sigma_raw = softplus_fast(o3);
        float4 out;
        out.x = sigmoid_fast(o0); out.y = sigmoid_fast(o1); out.z = sigmoid_fast(o2);
        out.w = (out_mode == kOutAlpha) ? (1.f - __expf(-(sigma_raw * r.decay))) : sigma_raw;
        rec_out[r.slot] = out;
        if (KEEP) rec_ext[r.slot] = make_float4(sigma_raw, o3, __uint_as_float(relu1), __uint_as_float(relu2));
      }
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
  }

  if (!ok) {
    if (tid == 0) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TIMEOUT);
    // our own bulk copy may still be in flight: give it a bounded chance to land before the CTA's
    // shared memory is released
    if (copy_pending) mbar_wait(bar_w, ph_w);
  }
  if (bad) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------ packing ----
__global__ void k_pack_weights(const float* __restrict__ W1, const float* __restrict__ b1, const float* __restrict__ W2,
                               const float* __restrict__ b2, const float* __restrict__ W3, const float* __restrict__ b3,
                               int n, char* __restrict__ out, int32_t* __restrict__ status) {
  const int p = blockIdx.x;
  if (p >= n) return;
  char* dst = out + (size_t)p * kWeightBytes;
  __half* w1 = reinterpret_cast<__half*>(dst + kOffW1);
  __half* w2 = reinterpret_cast<__half*>(dst + kOffW2);
  __half* w3 = reinterpret_cast<__half*>(dst + kOffW3);
  float* bias = reinterpret_cast<float*>(dst + kOffBias);
  bool bad = false;
  for (int i = threadIdx.x; i < kH * kK1; i += blockDim.x) {
    const int h = i / kK1, k = i % kK1;
    const __half v = __float2half_rn(k < 72 ? W1[(size_t)p * kH * 72 + h * 72 + k] : 0.f);
    bad |= __hisinf(v) || __hisnan(v);
    w1[(k >> 3) * (kH * 8) + h * 8 + (k & 7)] = v;
  }
  for (int i = threadIdx.x; i < kH * kH; i += blockDim.x) {
    const int h = i / kH, k = i % kH;
    const __half v = __float2half_rn(W2[(size_t)p * kH * kH + i]);
    bad |= __hisinf(v) || __hisnan(v);
    w2[(k >> 3) * (kH * 8) + h * 8 + (k & 7)] = v;
  }
  for (int i = threadIdx.x; i < kN3 * kH; i += blockDim.x) {
    const int h = i / kH, k = i % kH;
    const __half v = __float2half_rn(h < 4 ? W3[(size_t)p * 4 * kH + h * kH + k] : 0.f);
    bad |= __hisinf(v) || __hisnan(v);
    w3[(k >> 3) * (kN3 * 8) + h * 8 + (k & 7)] = v;
  }
  for (int i = threadIdx.x; i < kH; i += blockDim.x) {
    bias[i] = b1[(size_t)p * kH + i];
    bias[kH + i] = b2[(size_t)p * kH + i];
    bad |= !isfinite(bias[i]) || !isfinite(bias[kH + i]);
  }
  if (threadIdx.x < 4) { bias[2 * kH + threadIdx.x] = b3[(size_t)p * 4 + threadIdx.x]; bad |= !isfinite(bias[2 * kH + threadIdx.x]); }
  if (bad && status) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
}

int launch_mlp_f16(const mlpsp_scene* sc, const RecIn* rec_in, const int32_t* prim_off, const int2* work,
                   const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                   cudaStream_t st) {
  MLPSP_REQUIRE(sc->hidden == kH && sc->num_freq == 6, MLPSP_E_LIMIT,
                "fp16 evaluator is built for the 72->32->32->4 network (hidden 32, 6 frequencies)");
  MLPSP_REQUIRE(sc->w16 && sc->freq && sc->att, MLPSP_E_ARG, "fp16 evaluator needs the packed weight image");
  static bool attr_set = false;
  if (!attr_set) {
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // tensor memory: 512 columns per SM / 64 per CTA = at most 8 resident CTAs; shared memory and
  // registers (64 per thread) allow 7
  const int grid = sms * 7;
  LaunchScope scope(kKMlp, 1, st);
  if (rec_ext)
    k_mlp_tc<true><<<grid, kRows, kSmemBytes, st>>>((const char*)sc->w16, sc->freq, sc->att, rec_in, prim_off, work,
                                                   const_cast<int32_t*>(counters), rec_out, rec_ext, out_mode, status);
  else
    k_mlp_tc<false><<<grid, kRows, kSmemBytes, st>>>((const char*)sc->w16, sc->freq, sc->att, rec_in, prim_off, work,
                                                    const_cast<int32_t*>(counters), rec_out, rec_ext, out_mode, status);
  return cuda_check(cudaGetLastError(), "mlp_f16");
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int64_t mlpsp_packed_weight_bytes(int32_t hidden, int32_t num_freq) {
  return (hidden == kH && num_freq == 6) ? kWeightBytes : 0;
}

extern "C" int mlpsp_pack_weights_f16(const mlpsp_scene* sc, void* w16_out, int32_t* status, void* stream) {
  MLPSP_REQUIRE(sc && w16_out, MLPSP_E_ARG, "mlpsp_pack_weights_f16: null pointer");
  MLPSP_REQUIRE(sc->hidden == kH && sc->num_freq == 6, MLPSP_E_LIMIT,
                "mlpsp_pack_weights_f16: only the 72->32->32->4 network has a packed fp16 image");
  MLPSP_REQUIRE(sc->W1 && sc->b1 && sc->W2 && sc->b2 && sc->W3 && sc->b3, MLPSP_E_ARG,
                "mlpsp_pack_weights_f16: FP32 weights missing");
  if (sc->n == 0) return MLPSP_OK;
  LaunchScope scope(kKMisc, 1, (cudaStream_t)stream);
  k_pack_weights<<<sc->n, 128, 0, (cudaStream_t)stream>>>(sc->W1, sc->b1, sc->W2, sc->b2, sc->W3, sc->b3, sc->n,
                                                         (char*)w16_out, status);
  return cuda_check(cudaGetLastError(), "pack_weights_f16");
}
