// Per-primitive weight gradients of the 72-32-32-4 MLP on the 5th-generation tensor cores (tcgen05, sm_100a):
// the mixed-precision modes of grouped_weight_gradients (scannet/primitive_gemm.py:101-166: binary16 or bfloat16
// operands, FP32 accumulation over the whole segment, adjoints scaled before the cast and unscaled in FP32).
//
// One CTA owns one prepared segment of one primitive and walks it in blocks of 128 records (thread = record).
// All operand tiles of a block live in shared memory as chunks of [128 records][8 elements] (16 bytes per record,
// 2,048 bytes per chunk).  That one layout serves two kinds of product:
//   * record-major products (rows of D = records), the tile is the K-major A operand as in the evaluator:
//       H1 = relu(E W1^T + b1), H2 = relu(H1 W2^T + b2), D2 = (D3 W3) * mask2, D1 = (D2 W2) * mask1;
//   * the weight gradients contract over the records, so the same bytes are read as MN-major operands
//     (eight records x eight elements = one 128-byte core matrix with the element dimension contiguous):
//       dW1^T [72 x 32] += E^T D1,   dW2^T [32 x 32] += H1^T D2,   dW3^T [32 x 4] += H2^T D3
//     with M = 128 rows of the tensor core over the element dimension (rows past the operand's width read the
//     chunks that follow and land in accumulator lanes nobody looks at), N = 32 or 16, K = 16 records per MMA.
//     A chunk of ones directly behind E, H1 and H2 makes the bias gradients the next accumulator lane:
//     db1 = sum D1 is lane 72 of dW1^T, db2 / db3 lane 32 of dW2^T / dW3^T -- FP32 sums of the rounded adjoints,
//     as primitive_gemm.py:157-160 takes them.
// The three gradient accumulators stay in tensor memory for the whole segment and are written, divided by the
// scale, as the segment's partial row; k_reduce_partials (backward.cu) adds the rows of a primitive in order.
//
// A block costs five MMA round trips (layer 1, layer 2, D2, D1, gradients), each: operand tile complete ->
// fence -> CTA barrier -> one thread issues and commits -> everyone waits on the mbarrier (bounded: a wait that
// gives up sets bit 1 of the flag word and the CTA leaves after freeing its tensor memory).  The gradient MMAs
// of a block run while the threads compute the next block's encoding in registers.
#include "frame.cuh"
#include "tc.cuh"

namespace mlpsp {

constexpr int kVjpRows = 128, kVjpChunk = kVjpRows * 16;
// chunk indices of the operand tiles
constexpr int kVcE = 0, kVcOneE = 9, kVcH1 = 10, kVcOneH1 = 14, kVcH2 = 15, kVcOneH2 = 19, kVcD1 = 20, kVcD2 = 24,
              kVcD3 = 28, kVcEnd = 30;
// weight operands (K-major B: [K / 8 chunks][32 rows][8 elements], 512 bytes per chunk)
constexpr int kVoW1 = kVcEnd * kVjpChunk;          // W1[h][j], 10 chunks (the last one zero: it meets the ones behind E)
constexpr int kVoW2 = kVoW1 + 10 * 512;            // W2[q][h], 4 chunks
constexpr int kVoW2T = kVoW2 + 4 * 512;            // rows h, K = q: W2[q][h]
constexpr int kVoW3T = kVoW2T + 4 * 512;           // rows h, K = output c (4 of 16): W3[c][h]
constexpr int kVoBias = kVoW3T + 2 * 512;          // b1[32], b2[32] as FP32
constexpr int kVoBar = kVoBias + 256;
constexpr int kVjpSmem = kVoBar + 16;
constexpr int kVjpTmemCols = 128;                  // [0,32) transient, [32,64) dW1^T, [64,96) dW2^T, [96,112) dW3^T
static_assert((kVcH2 + 16) * kVjpChunk <= kVoW2, "an M = 128 window from any tile start stays inside the allocation");

constexpr int kVW1 = 32 * 72, kVW2 = 32 * 32, kVW3 = 4 * 32;
constexpr int kVOb1 = kVW1, kVOW2 = kVOb1 + 32, kVOb2 = kVOW2 + kVW2, kVOW3 = kVOb2 + 32, kVOb3 = kVOW3 + kVW3;
static_assert(kVOb3 + 4 == 3524, "gradient row layout");

// instruction descriptor with both operands MN-major (bits 15 and 16)
__host__ __device__ constexpr uint32_t vjp_idesc_mn(int M, int N, bool bf16) { return instr_desc(M, N, bf16) | (1u << 15) | (1u << 16); }

template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(pack_h2<BF16>(v[0], v[1]), pack_h2<BF16>(v[2], v[3]), pack_h2<BF16>(v[4], v[5]), pack_h2<BF16>(v[6], v[7]));
}

template <bool BF16>
__global__ void __launch_bounds__(kVjpRows, 3) k_grouped_vjp_tc(
    const float* __restrict__ x6, const float* __restrict__ d4, const int32_t* __restrict__ masks,
    const int64_t* __restrict__ offsets, const int64_t* __restrict__ seg_prim, const int64_t* __restrict__ seg_start,
    int segment_size, const float* __restrict__ freq, const float* __restrict__ att, const float* __restrict__ W1,
    const float* __restrict__ b1, const float* __restrict__ W2, const float* __restrict__ b2,
    const float* __restrict__ W3, float scale, float* __restrict__ partial, int32_t* __restrict__ flag) {
  extern __shared__ __align__(128) char smem[];
  const int seg = blockIdx.x, tid = threadIdx.x, warp = tid >> 5;
  const int p = (int)seg_prim[seg];
  const int64_t begin = seg_start[seg];
  const int total = (int)min((int64_t)segment_size, offsets[p + 1] - begin);
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + kVoBar);
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 1);
  float* s_b1 = reinterpret_cast<float*>(smem + kVoBias);
  float* s_b2 = s_b1 + 32;
  const uint32_t sb = smem_u32(smem), bar = smem_u32(s_bar);
  if (tid == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_misc[0]), kVjpTmemCols);
  // tiles: zeros, except the three chunks of ones
  {
    const uint32_t one2 = BF16 ? 0x3f803f80u : 0x3c003c00u;
    for (int i = tid; i < kVcEnd * kVjpRows; i += kVjpRows) {
      const int chunk = i >> 7;
      const uint32_t v = (chunk == kVcOneE || chunk == kVcOneH1 || chunk == kVcOneH2) ? one2 : 0u;
      *reinterpret_cast<uint4*>(smem + (size_t)i * 16) = make_uint4(v, v, v, v);
    }
  }
  // the primitive's weights in the operand format (RN), as primitive_gemm.py:118-120 casts them
  {
    const float* w1 = W1 + (size_t)p * kVW1;
    const float* w2 = W2 + (size_t)p * kVW2;
    const float* w3 = W3 + (size_t)p * kVW3;
    float v[8];
    for (int g = tid; g < 320; g += kVjpRows) {
      const int n = g & 31, kc = g >> 5;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = kc < 9 ? __ldg(w1 + n * 72 + kc * 8 + i) : 0.f;
      *reinterpret_cast<uint4*>(smem + kVoW1 + kc * 512 + n * 16) = pack8<BF16>(v);
    }
    {
      const int n = tid & 31, kc = tid >> 5;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __ldg(w2 + n * 32 + kc * 8 + i);
      *reinterpret_cast<uint4*>(smem + kVoW2 + kc * 512 + n * 16) = pack8<BF16>(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __ldg(w2 + (kc * 8 + i) * 32 + n);
      *reinterpret_cast<uint4*>(smem + kVoW2T + kc * 512 + n * 16) = pack8<BF16>(v);
    }
    if (tid < 64) {
      const int n = tid & 31, kc = tid >> 5;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (kc == 0 && i < 4) ? __ldg(w3 + i * 32 + n) : 0.f;
      *reinterpret_cast<uint4*>(smem + kVoW3T + kc * 512 + n * 16) = pack8<BF16>(v);
    }
    if (tid < 32) { s_b1[tid] = __ldg(b1 + (size_t)p * 32 + tid); s_b2[tid] = __ldg(b2 + (size_t)p * 32 + tid); }
  }
  float mult[6];
#pragma unroll
  for (int f = 0; f < 6; ++f) mult[f] = __ldg(freq + f) * __ldg(att + f);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);

  const uint32_t idesc_h = instr_desc(kVjpRows, 32, BF16);
  const uint32_t idesc_g32 = vjp_idesc_mn(kVjpRows, 32, BF16), idesc_g16 = vjp_idesc_mn(kVjpRows, 16, BF16);
  auto tile = [&](int chunk) { return sb + (uint32_t)chunk * kVjpChunk; };
  // record-major A operand (K-major): K chunks a chunk apart, groups of eight records 128 bytes apart
  auto a_rows = [&](int chunk) { return smem_desc(tile(chunk), kVjpChunk, 128); };
  // K-major B operand of the weights
  auto b_w = [&](int off) { return smem_desc(sb + off, 512, 128); };
  // MN-major operand: groups of eight elements a chunk apart, groups of eight records 128 bytes apart
  auto mn = [&](int chunk) { return smem_desc(tile(chunk), 128, kVjpChunk); };
  auto adv = [](uint64_t desc, int bytes) { return desc + (uint64_t)(bytes >> 4); };

  char* my = smem + tid * 16;
  uint32_t ph = 0u;
  bool ok = true;
  // tile writes visible to the tensor core, tensor-memory reads retired, then one thread issues and commits
  auto issue_phase = [&](auto issue) {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue();
      mma_commit(bar);
    }
  };
  auto wait_phase = [&]() -> bool {
    const bool done = mbar_wait(bar, ph & 1u);
    ++ph;
    tc_fence_after();
    return __syncthreads_and(done) != 0;
  };
  auto round_trip = [&](auto issue) -> bool {
    issue_phase(issue);
    return wait_phase();
  };
  bool grads_pending = false;     // the previous block's gradient MMAs still read its tiles

  for (int sub = 0; sub < total && ok; sub += kVjpRows) {
    const int cnt = min(kVjpRows, total - sub);
    const bool valid = tid < cnt;
    const int64_t r = begin + sub + tid;
    uint32_t m1 = 0u, m2 = 0u;
    // ---- encoding (index c * 6 + f holds sin, 36 + c * 6 + f holds cos: scannet/cumodel.py:183-195) and D3,
    //      into registers while the previous block's gradient MMAs finish ----
    uint32_t ew[36];                                            // 32-bit word = two consecutive encoding entries
#pragma unroll
    for (int c = 0; c < 6; ++c) {
      float sn[6], cs[6];
      const float v = valid ? __ldg(x6 + r * 6 + c) : 0.f;
#pragma unroll
      for (int f = 0; f < 6; ++f) {
        if (valid) __sincosf(v * mult[f], &sn[f], &cs[f]);
        else { sn[f] = 0.f; cs[f] = 0.f; }
      }
#pragma unroll
      for (int g = 0; g < 3; ++g) {
        ew[3 * c + g] = pack_h2<BF16>(sn[2 * g], sn[2 * g + 1]);
        ew[18 + 3 * c + g] = pack_h2<BF16>(cs[2 * g], cs[2 * g + 1]);
      }
    }
    float4 g4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      g4 = __ldg(reinterpret_cast<const float4*>(d4) + r);
      if (masks) { m1 = (uint32_t)__ldg(masks + r * 2); m2 = (uint32_t)__ldg(masks + r * 2 + 1); }
    }
    if (grads_pending) {
      ok = wait_phase();
      grads_pending = false;
      if (!ok) break;
    }
#pragma unroll
    for (int kc = 0; kc < 9; ++kc)
      *reinterpret_cast<uint4*>(my + (kVcE + kc) * kVjpChunk) = make_uint4(ew[4 * kc], ew[4 * kc + 1], ew[4 * kc + 2], ew[4 * kc + 3]);
    *reinterpret_cast<uint4*>(my + kVcD3 * kVjpChunk) =
        make_uint4(pack_h2<BF16>(g4.x * scale, g4.y * scale), pack_h2<BF16>(g4.z * scale, g4.w * scale), 0u, 0u);
    // ---- layer 1: K = 80 (the ones behind E meet the zero chunk of W1) ----
    ok = round_trip([&]() {
      const uint64_t a = a_rows(kVcE), b = b_w(kVoW1);
#pragma unroll
      for (int ks = 0; ks < 5; ++ks) mma_f16(tmem, adv(a, ks * 2 * kVjpChunk), adv(b, ks * 2 * 512), idesc_h, ks > 0);
    });
    if (!ok) break;
    {
      uint32_t acc[32];
      tmem_ld32(trow, acc);
      uint32_t sign = 0u;
#pragma unroll
      for (int kc = 0; kc < 4; ++kc) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = kc * 8 + q * 2;
          const float v0 = __uint_as_float(acc[j]) + s_b1[j], v1 = __uint_as_float(acc[j + 1]) + s_b1[j + 1];
          sign |= (v0 > 0.f ? 1u : 0u) << j;
          sign |= (v1 > 0.f ? 1u : 0u) << (j + 1);
          w[q] = pack_h2_relu<BF16>(v0, v1);
        }
        *reinterpret_cast<uint4*>(my + (kVcH1 + kc) * kVjpChunk) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (!masks) m1 = sign;
    }
    // ---- layer 2 ----
    ok = round_trip([&]() {
      const uint64_t a = a_rows(kVcH1), b = b_w(kVoW2);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) mma_f16(tmem, adv(a, ks * 2 * kVjpChunk), adv(b, ks * 2 * 512), idesc_h, ks > 0);
    });
    if (!ok) break;
    {
      uint32_t acc[32];
      tmem_ld32(trow, acc);
      uint32_t sign = 0u;
#pragma unroll
      for (int kc = 0; kc < 4; ++kc) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = kc * 8 + q * 2;
          const float v0 = __uint_as_float(acc[j]) + s_b2[j], v1 = __uint_as_float(acc[j + 1]) + s_b2[j + 1];
          sign |= (v0 > 0.f ? 1u : 0u) << j;
          sign |= (v1 > 0.f ? 1u : 0u) << (j + 1);
          w[q] = pack_h2_relu<BF16>(v0, v1);
        }
        *reinterpret_cast<uint4*>(my + (kVcH2 + kc) * kVjpChunk) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (!masks) m2 = sign;
    }
    // ---- D2 = (D3 W3) * mask2: K = 16 ----
    ok = round_trip([&]() { mma_f16(tmem, a_rows(kVcD3), b_w(kVoW3T), idesc_h, 0u); });
    if (!ok) break;
    {
      uint32_t acc[32];
      tmem_ld32(trow, acc);
#pragma unroll
      for (int kc = 0; kc < 4; ++kc) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = kc * 8 + q * 2;
          const float v0 = ((m2 >> j) & 1u) ? __uint_as_float(acc[j]) : 0.f;
          const float v1 = ((m2 >> (j + 1)) & 1u) ? __uint_as_float(acc[j + 1]) : 0.f;
          w[q] = pack_h2<BF16>(v0, v1);
        }
        *reinterpret_cast<uint4*>(my + (kVcD2 + kc) * kVjpChunk) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    // ---- D1 = (D2 W2) * mask1: K = 32 ----
    ok = round_trip([&]() {
      const uint64_t a = a_rows(kVcD2), b = b_w(kVoW2T);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) mma_f16(tmem, adv(a, ks * 2 * kVjpChunk), adv(b, ks * 2 * 512), idesc_h, ks > 0);
    });
    if (!ok) break;
    {
      uint32_t acc[32];
      tmem_ld32(trow, acc);
#pragma unroll
      for (int kc = 0; kc < 4; ++kc) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = kc * 8 + q * 2;
          const float v0 = ((m1 >> j) & 1u) ? __uint_as_float(acc[j]) : 0.f;
          const float v1 = ((m1 >> (j + 1)) & 1u) ? __uint_as_float(acc[j + 1]) : 0.f;
          w[q] = pack_h2<BF16>(v0, v1);
        }
        *reinterpret_cast<uint4*>(my + (kVcD1 + kc) * kVjpChunk) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    // ---- gradients: contraction over the block's 128 records, 16 per MMA ----
    const uint32_t keep = sub > 0 ? 1u : 0u;
    issue_phase([&]() {
      const uint64_t e = mn(kVcE), h1 = mn(kVcH1), h2 = mn(kVcH2), d1 = mn(kVcD1), d2 = mn(kVcD2), d3 = mn(kVcD3);
#pragma unroll
      for (int ks = 0; ks < kVjpRows / 16; ++ks) {
        const uint32_t acc = (keep || ks > 0) ? 1u : 0u;
        mma_f16(tmem + 32, adv(e, ks * 256), adv(d1, ks * 256), idesc_g32, acc);
        mma_f16(tmem + 64, adv(h1, ks * 256), adv(d2, ks * 256), idesc_g32, acc);
        mma_f16(tmem + 96, adv(h2, ks * 256), adv(d3, ks * 256), idesc_g16, acc);
      }
    });
    grads_pending = true;
  }
  if (ok && grads_pending) ok = wait_phase();

  if (ok) {
    float* out = partial + (size_t)seg * 3524;
    const float inv = 1.f / scale;
    uint32_t acc[32];
    tmem_ld32(trow + 32, acc);                       // lane j of dW1^T: dW1[h][j] for the 32 h; lane 72: db1
    if (tid < 72) {
#pragma unroll
      for (int h = 0; h < 32; ++h) out[h * 72 + tid] = __uint_as_float(acc[h]) * inv;
    } else if (tid == 72) {
#pragma unroll
      for (int h = 0; h < 32; ++h) out[kVOb1 + h] = __uint_as_float(acc[h]) * inv;
    }
    if (warp < 2) {                                  // lanes 0..31: dW2[q][h = lane], dW3[c][h = lane]; lane 32: db2, db3
      tmem_ld32(trow + 64, acc);
      uint32_t o3[4];
      tmem_ld4(trow + 96, o3);
      if (tid < 32) {
#pragma unroll
        for (int q = 0; q < 32; ++q) out[kVOW2 + q * 32 + tid] = __uint_as_float(acc[q]) * inv;
#pragma unroll
        for (int c = 0; c < 4; ++c) out[kVOW3 + c * 32 + tid] = __uint_as_float(o3[c]) * inv;
      } else if (tid == 32) {
#pragma unroll
        for (int q = 0; q < 32; ++q) out[kVOb2 + q] = __uint_as_float(acc[q]) * inv;
#pragma unroll
        for (int c = 0; c < 4; ++c) out[kVOb3 + c] = __uint_as_float(o3[c]) * inv;
      }
    }
  } else if (tid == 0) {
    atomicOr(flag, 2);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, kVjpTmemCols);
}

int launch_grouped_vjp_tc(bool bf16, const float* x6, const float* d4, const int32_t* masks, const int64_t* offsets,
                          const int64_t* seg_prim, const int64_t* seg_start, int64_t num_segments, int segment_size,
                          const mlpsp_scene* sc, float scale, float* partial, int32_t* flag, cudaStream_t st) {
  static DeviceOnce attr_once;
  if (attr_once.first()) {
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_grouped_vjp_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kVjpSmem));
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_grouped_vjp_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kVjpSmem));
  }
  if (bf16)
    k_grouped_vjp_tc<true><<<(unsigned)num_segments, kVjpRows, kVjpSmem, st>>>(x6, d4, masks, offsets, seg_prim, seg_start, segment_size,
                                                                             sc->freq, sc->att, sc->W1, sc->b1, sc->W2, sc->b2,
                                                                             sc->W3, scale, partial, flag);
  else
    k_grouped_vjp_tc<false><<<(unsigned)num_segments, kVjpRows, kVjpSmem, st>>>(x6, d4, masks, offsets, seg_prim, seg_start, segment_size,
                                                                              sc->freq, sc->att, sc->W1, sc->b1, sc->W2, sc->b2,
                                                                              sc->W3, scale, partial, flag);
  return cuda_check(cudaGetLastError(), "grouped_vjp_tc");
}

}  // namespace mlpsp
