// Gated feature compositing as a contraction on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   out_feat[pix, :] = sum over the pixel's composited records of w * mix(p, gates)          (np_tile_kernels.cu:6036-6075)
// with mix = sum_s g_s attr[p, s, :] (S = 4), attr[p, 0, :] + sum_s g_s attr[p, 1+s, :] (S = 5) or attr[p, 0, :] (S = 1).
// The reference adds C values to global memory per hit.  Per tile this is a product
//   D^T [C x 64 pixels] = Attr^T [C x K] . Coef [K x 64 pixels],   K = (touched primitives of the tile) x S,
// where Coef holds w * g_s of the consumed (pixel, primitive) records and zeros elsewhere.  One CTA owns one
// (tile, block of 128 or 256 channels) and walks the tile's touched primitives 16 at a time:
//   * the attribute rows (binary16, the reference's inference storage format, scannet/checkpoints.py:358-359) are
//     gathered from this GPU's memory with cp.async into the MN-major core-matrix layout (eight K rows of eight
//     channels = 128 bytes) that tcgen05.mma reads as its A operand: the channel dimension is M, so all 128 rows
//     of the tensor core carry channels;
//   * every thread turns four (pixel, primitive) cells into coefficients: weight and gates of the record when the
//     pixel composited the primitive, zero otherwise, split into a binary16 head and a binary16 tail so that the
//     two products together carry 22 mantissa bits (the attributes themselves are exact);
//   * one thread issues the MMAs of the stage (128 x 64 x 16 each, FP32 accumulators in tensor memory) and commits
//     them to the mbarrier that guards the stage's buffers; the other stage is filled meanwhile.
// The copies and the record loads of the next stage are in flight while a stage is finished.
// Afterwards each warp reads its 32 channels x 64 pixels from tensor memory and writes 128-byte lines of the map.
//
// Every wait on an mbarrier is bounded (MLPSP_ST_TIMEOUT), copies in flight are waited for, tensor memory is freed.
#include "frame.cuh"
#include "tc.cuh"

namespace mlpsp {

constexpr int kFtThreads = 256;
constexpr int kFtPairs = 16;          // touched primitives per stage
constexpr int kFtListMax = 2048;      // candidates of a tile the kernel looks at (kWinMax of the wave kernels)
constexpr int kFtMeta = 256;          // touched primitives whose masks and bases are held in shared memory at a time

// what the kernel needs of one touched (tile, primitive) pair
struct __align__(8) FtMeta {
  int32_t prim;
  uint32_t base;     // compositing slot of the pair's first record
  uint32_t u0, u1;   // pixels that composited the primitive
  uint32_t m0, m1;   // pixels whose hit was evaluated (the record's slot is its rank among them)
};
static_assert(sizeof(FtMeta) == 24, "shared-memory plan");

__device__ __forceinline__ void ft_cp_async16(uint32_t dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;   // source size 0: the 16 bytes are written as zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ft_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// instruction descriptor: D = F32, A = B = F16, A MN-major (bit 15), B K-major, dense
__host__ __device__ constexpr uint32_t ft_instr_desc(int M, int N) {
  return (1u << 4) | (1u << 15) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// shared memory of one stage: A [K/8 groups of eight K rows][CB/8 groups of eight channels][8 rows][8 halves],
// then the coefficient heads and tails [K/8 chunks][64 pixels][8 halves] each
template <int S>
struct FtPlan {
  static constexpr int K = kFtPairs * S;                       // 16 / 64 / 80, a multiple of the MMA's K = 16
  __host__ __device__ static constexpr int a_bytes(int CB) { return K * CB * 2; }
  static constexpr int kCoefBytes = 64 * K * 2;
  __host__ __device__ static constexpr int stage_bytes(int CB) { return a_bytes(CB) + 2 * kCoefBytes; }
  __host__ __device__ static constexpr int smem_bytes(int CB) { return 2 * stage_bytes(CB) + 2 * kFtListMax + kFtMeta * 24 + 64; }
};

template <int S>
__global__ void __launch_bounds__(kFtThreads, 2) k_feature_tc(
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ tile_len, const int32_t* __restrict__ sorted_prims,
    int W, int H, int ntx, const uint32_t* __restrict__ used32, const uint32_t* __restrict__ masks32,
    const uint32_t* __restrict__ pair_base, const float* __restrict__ rec_w, const float4* __restrict__ rec_gate,
    const __half* __restrict__ feat16, int C, int CB, float* __restrict__ out_feat, int32_t* __restrict__ status) {
  using P = FtPlan<S>;
  constexpr int K = P::K;
  extern __shared__ __align__(128) char smem[];
  __shared__ int warp_sums[32];
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tile = blockIdx.x, c0 = blockIdx.y * CB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int stage_bytes = P::stage_bytes(CB);
  uint16_t* s_idx = reinterpret_cast<uint16_t*>(smem + 2 * stage_bytes);            // touched candidates of the tile
  FtMeta* s_meta = reinterpret_cast<FtMeta*>(smem + 2 * stage_bytes + 2 * kFtListMax);
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + 2 * stage_bytes + 2 * kFtListMax + kFtMeta * 24);   // [0..1] MMAs of a stage buffer done
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 2);                        // [0] tmem base
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar0 = smem_u32(&s_bar[0]);
  const int nb128 = CB / 128;
  const uint32_t tmem_cols = nb128 == 2 ? 128u : 64u;
  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_misc[0]), tmem_cols);

  // ---- the tile's touched candidates (some pixel composited the primitive), in list order ----
  const int s = tile_offsets[tile];
  const int len = min(tile_len[tile], kFtListMax);
  int nt = 0;
  for (int j0 = 0; j0 < len; j0 += kFtThreads) {
    const int j = j0 + tid;
    bool touched = false;
    if (j < len) {
      const uint2 u = *reinterpret_cast<const uint2*>(used32 + 2 * (size_t)(s + j));
      touched = (u.x | u.y) != 0u;
    }
    int total;
    const int pos = block_exclusive_scan(touched ? 1 : 0, warp_sums, total);
    if (touched) s_idx[nt + pos] = (uint16_t)j;
    nt += total;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  const int a_bytes = P::a_bytes(CB);
  const uint32_t lbo_a = (uint32_t)CB * 16u;      // between groups of eight K rows
  const uint32_t idesc = ft_instr_desc(128, 64);
  bool ok = true;
  int gs = 0;                                     // stages issued so far: buffer = gs & 1, use of that buffer = gs >> 1
  const int px = tid & 63;

  // the MMAs that last read the buffer of stage g (two stages earlier) have finished
  auto buffer_free = [&](int g) {
    if (g >= 2) ok = mbar_wait(bar0 + 8 * (g & 1), (uint32_t)((g >> 1) - 1) & 1u) && ok;
  };
  // Attribute rows of the 16 primitives from touched index t0 on (batch-local index l0): a warp copies eight K rows x
  // four channel groups at a time, so that eight lanes fill one 128-byte core matrix (no bank conflicts) and four
  // lanes read 64 contiguous bytes.  One cp.async group per stage.
  auto issue_copies = [&](int g, int l0, int nb) {
    const uint32_t a_s = sb + (g & 1) * stage_bytes;
    const int gq_n = CB / 32;
    for (int task = warp; task < (K / 8) * gq_n; task += kFtThreads / 32) {
      const int kg = task / gq_n, gq = task - kg * gq_n;
      const int k = kg * 8 + (lane & 7), grp = gq * 4 + (lane >> 3);
      const int pl = k / S, sl = k - pl * S;
      const bool valid = l0 + pl < nb;
      const int prim = valid ? s_meta[l0 + pl].prim : 0;
      const __half* src = feat16 + ((size_t)prim * S + sl) * C + c0 + grp * 8;
      ft_cp_async16(a_s + kg * lbo_a + grp * 128 + (lane & 7) * 16, src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // weight and gates of this thread's four (pixel, primitive) cells of a stage; zero where the pixel did not
  // composite the primitive
  auto load_cells = [&](int l0, int nb, float (&cw)[kFtPairs / 4], float4 (&cg)[kFtPairs / 4]) {
#pragma unroll
    for (int i = 0; i < kFtPairs / 4; ++i) {
      const int l = l0 + (tid >> 6) + 4 * i;
      cw[i] = 0.f;
      cg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (l < nb) {
        const FtMeta m = s_meta[l];
        const uint32_t u = px < 32 ? m.u0 : m.u1;
        if ((u >> (px & 31)) & 1u) {
          const uint32_t slot = m.base + (px < 32 ? __popc(m.m0 & ((1u << px) - 1u))
                                                  : __popc(m.m0) + __popc(m.m1 & ((1u << (px - 32)) - 1u)));
          cw[i] = __ldg(rec_w + slot);
          if (S > 1) cg[i] = __ldg(rec_gate + slot);
        }
      }
    }
  };
  // coefficients of the cells, head + tail in binary16; K index of slot sl of the stage's primitive pl is pl * S + sl,
  // element (pixel, k) sits at (k / 8) * 1024 + pixel * 16 + (k % 8) * 2
  auto write_coefs = [&](int g, const float (&cw)[kFtPairs / 4], const float4 (&cg)[kFtPairs / 4]) {
    char* coef_hi = smem + (g & 1) * stage_bytes + a_bytes;
    char* coef_lo = coef_hi + P::kCoefBytes;
#pragma unroll
    for (int i = 0; i < kFtPairs / 4; ++i) {
      const int pl = (tid >> 6) + 4 * i;
      const float w = cw[i];
      float cf[5];
      if (S == 1) { cf[0] = w; }
      else if (S == 4) { cf[0] = w * cg[i].x; cf[1] = w * cg[i].y; cf[2] = w * cg[i].z; cf[3] = w * cg[i].w; }
      else { cf[0] = w; cf[1] = w * cg[i].x; cf[2] = w * cg[i].y; cf[3] = w * cg[i].z; cf[4] = w * cg[i].w; }
      __half hi[5], lo[5];
#pragma unroll
      for (int sl = 0; sl < S; ++sl) {
        hi[sl] = __float2half_rn(cf[sl]);
        lo[sl] = __float2half_rn(cf[sl] - __half2float(hi[sl]));
      }
      if (S == 4) {
        const int off = (pl >> 1) * 1024 + px * 16 + (pl & 1) * 8;
        *reinterpret_cast<uint2*>(coef_hi + off) = make_uint2((uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[1]) << 16),
                                                              (uint32_t)__half_as_ushort(hi[2]) | ((uint32_t)__half_as_ushort(hi[3]) << 16));
        *reinterpret_cast<uint2*>(coef_lo + off) = make_uint2((uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[1]) << 16),
                                                              (uint32_t)__half_as_ushort(lo[2]) | ((uint32_t)__half_as_ushort(lo[3]) << 16));
      } else {
#pragma unroll
        for (int sl = 0; sl < S; ++sl) {
          const int k = pl * S + sl;
          const int off = (k >> 3) * 1024 + px * 16 + (k & 7) * 2;
          *reinterpret_cast<__half*>(coef_hi + off) = hi[sl];
          *reinterpret_cast<__half*>(coef_lo + off) = lo[sl];
        }
      }
    }
  };

  for (int b0 = 0; b0 < nt && ok; b0 += kFtMeta) {
    const int nb = min(kFtMeta, nt - b0);
    // ---- the batch's primitives, consumed masks, hit masks and record bases ----
    __syncthreads();
    for (int l = tid; l < nb; l += kFtThreads) {
      const size_t pi = (size_t)(s + s_idx[b0 + l]);
      const uint2 u = *reinterpret_cast<const uint2*>(used32 + 2 * pi), m = *reinterpret_cast<const uint2*>(masks32 + 2 * pi);
      FtMeta e;
      e.prim = __ldg(sorted_prims + pi); e.base = __ldg(pair_base + pi); e.u0 = u.x; e.u1 = u.y; e.m0 = m.x; e.m1 = m.y;
      s_meta[l] = e;
    }
    __syncthreads();
    // ---- stages of 16 primitives; the copies and the record loads of stage l+1 are in flight while stage l is
    // finished and handed to the tensor cores ----
    const int nsb = (nb + kFtPairs - 1) / kFtPairs;
    float cw[kFtPairs / 4];
    float4 cg[kFtPairs / 4];
    buffer_free(gs);
    issue_copies(gs, 0, nb);
    load_cells(0, nb, cw, cg);
    for (int ls = 0; ls < nsb; ++ls) {
      const int g = gs + ls;
      const bool more = ls + 1 < nsb;
      if (more) {
        buffer_free(g + 1);
        issue_copies(g + 1, (ls + 1) * kFtPairs, nb);
      }
      write_coefs(g, cw, cg);
      if (more) load_cells((ls + 1) * kFtPairs, nb, cw, cg);
      if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_async_smem();
      tc_fence_before();
      if (!__syncthreads_and(ok)) { ok = false; break; }
      if (tid == 0) {
        tc_fence_after();
        const uint32_t a_s = sb + (g & 1) * stage_bytes;
        const uint32_t hi_s = a_s + a_bytes, lo_s = hi_s + P::kCoefBytes;
        const uint64_t bh_desc = smem_desc(hi_s, 1024, 128), bl_desc = smem_desc(lo_s, 1024, 128);
        for (int h = 0; h < nb128; ++h) {
          // A: MN-major, 128 channels = 16 groups of eight (128 bytes apart), K groups of eight lbo_a apart
          const uint64_t a_desc = smem_desc(a_s + h * 2048, lbo_a, 128);
#pragma unroll
          for (int ks = 0; ks < K / 16; ++ks) {
            const uint64_t a_k = a_desc + (uint64_t)((ks * 2 * lbo_a) >> 4);
            mma_f16(tmem + h * 64, a_k, bh_desc + (uint64_t)((ks * 2 * 1024) >> 4), idesc, (g > 0 || ks > 0) ? 1u : 0u);
            mma_f16(tmem + h * 64, a_k, bl_desc + (uint64_t)((ks * 2 * 1024) >> 4), idesc, 1u);
          }
        }
        mma_commit(bar0 + 8 * (g & 1));
      }
    }
    gs += nsb;
  }
  const int nst = gs;

  // ---- the last stage's MMAs (tensor-core instructions complete in order) ----
  if (ok && nst > 0) {
    const int last = nst - 1;
    ok = mbar_wait(bar0 + 8 * (last & 1), (uint32_t)(last >> 1) & 1u);
  }
  ok = __all_sync(0xffffffffu, ok);
  tc_fence_after();
  // ---- epilogue: warp = 32 channels of one 128-channel half, thread = channel, 64 pixels from tensor memory ----
  const int q = warp & 3, h = warp >> 2;
  if (h < nb128) {
    const int c = c0 + h * 128 + q * 32 + lane;
    const int x0 = (tile % ntx) * 8, y0 = (tile / ntx) * 8;
#pragma unroll 1
    for (int part = 0; part < 2; ++part) {
      uint32_t v[32];
      if (ok && nst > 0) {
        tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + h * 64 + part * 32, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int x = x0 + (i & 7), y = y0 + part * 4 + (i >> 3);      // pixel part * 32 + i of the tile
        if (x < W && y < H) out_feat[((size_t)y * W + x) * C + c] = __uint_as_float(v[i]);
      }
    }
  }
  if (!ok) {
    if (tid == 0) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TIMEOUT);
    ft_cp_async_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, tmem_cols);
}

// binary16 copy of the attributes [n, S, C]; raises MLPSP_ST_FEAT_INEXACT when a value does not survive the round trip
__global__ void k_pack_features(const float* __restrict__ attr, int64_t count, __half* __restrict__ out, int32_t* __restrict__ status) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool inexact = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    const float v = attr[i];
    const __half hv = __float2half_rn(v);
    out[i] = hv;
    inexact |= !(__half2float(hv) == v);
  }
  if (inexact && status) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_FEAT_INEXACT);
}

bool feature_tc_supported(const mlpsp_scene* sc) {
  return sc->feat16 != nullptr && sc->feat_dim >= 128 && sc->feat_dim <= 512 && sc->feat_dim % 128 == 0 &&
         (sc->feat_slots == 1 || sc->feat_slots == 4 || sc->feat_slots == 5) &&
         (reinterpret_cast<uintptr_t>(sc->feat16) & 15) == 0;
}

template <int S>
static int launch_ft(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, const uint32_t* used32, int T, int ntx,
                     cudaStream_t st) {
  const int C = sc->feat_dim;
  const int CB = (C % 256 == 0) ? 256 : 128;
  const int smem = FtPlan<S>::smem_bytes(CB);
  static DeviceOnce attr_once;
  if (attr_once.first())
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_feature_tc<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, FtPlan<S>::smem_bytes(256)));
  const dim3 grid(T, C / CB);
  k_feature_tc<S><<<grid, kFtThreads, smem, st>>>(fr->tile_offsets, s.tile_len, fr->sorted_prims, fr->width, fr->height, ntx, used32,
                                                  s.masks32, s.pair_base, s.rec_w, s.rec_gate, (const __half*)sc->feat16, C, CB,
                                                  fr->feat, fr->status);
  return cuda_check(cudaGetLastError(), "feature_tc");
}

int launch_feature_tc(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, const uint32_t* used32, cudaStream_t st) {
  const int T = num_tiles(fr->width, fr->height, 8), ntx = (fr->width + 7) / 8;
  if (sc->feat_slots == 1) return launch_ft<1>(sc, fr, s, used32, T, ntx, st);
  if (sc->feat_slots == 4) return launch_ft<4>(sc, fr, s, used32, T, ntx, st);
  return launch_ft<5>(sc, fr, s, used32, T, ntx, st);
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int mlpsp_pack_features_f16(const mlpsp_scene* sc, void* feat16_out, int32_t* status, void* stream) {
  MLPSP_REQUIRE(sc && feat16_out, MLPSP_E_ARG, "mlpsp_pack_features_f16: null pointer");
  MLPSP_REQUIRE(sc->feat_attr && sc->feat_dim > 0 && sc->feat_slots > 0 && sc->n >= 0, MLPSP_E_ARG,
                "mlpsp_pack_features_f16: the scene has no feature attributes");
  const int64_t count = (int64_t)sc->n * sc->feat_slots * sc->feat_dim;
  if (count == 0) return MLPSP_OK;
  cudaStream_t st = (cudaStream_t)stream;
  LaunchScope scope(kKMisc, 1, st);
  const int blocks = (int)std::min<int64_t>((count + 255) / 256, 148 * 32);
  k_pack_features<<<blocks, 256, 0, st>>>(sc->feat_attr, count, (__half*)feat16_out, status);
  return cuda_check(cudaGetLastError(), "mlpsp_pack_features_f16");
}
