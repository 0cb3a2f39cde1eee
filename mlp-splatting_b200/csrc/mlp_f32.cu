// Scalar FP32 per-primitive evaluator: positional encoding + 12F -> H -> H -> 4 MLP in the
// operation order of the reference's scalar kernels (scannet/cuda/np_tile_kernels.cu:2047-2103):
// layer 1 starts from the bias and accumulates (sin weight, cos weight) per (component, frequency);
// layers 2 and 3 start from the bias and accumulate over ascending input index.
// One CTA per work item (primitive, up to 128 of its records); the primitive's FP32 weights are
// staged once in shared memory and every thread evaluates one record.
#include "frame.cuh"

namespace mlpsp {

template <int HMAX>
__global__ void __launch_bounds__(kRowsPerItem) k_mlp_f32(
    const float* __restrict__ W1, const float* __restrict__ b1, const float* __restrict__ W2,
    const float* __restrict__ b2, const float* __restrict__ W3, const float* __restrict__ b3,
    const float* __restrict__ freq, const float* __restrict__ att, int F, int H,
    const RecIn* __restrict__ rec_in, const int32_t* __restrict__ prim_off, const int4* __restrict__ work,
    int32_t* __restrict__ counters, float4* __restrict__ rec_out, float4* __restrict__ rec_ext, int out_mode,
    const int32_t* __restrict__ status) {
  extern __shared__ float sW[];
  __shared__ int s_item;
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int IN = 12 * F, half = 6 * F;
  float* sW1 = sW;
  float* sb1 = sW1 + H * IN;
  float* sW2 = sb1 + H;
  float* sb2 = sW2 + H * H;
  float* sW3 = sb2 + H;
  float* sb3 = sW3 + 4 * H;
  float* sfa = sb3 + 4;  // freq[f]*att is NOT pre-multiplied: the product is v*freq*att left to right
  const int tid = threadIdx.x;
  const int G = counters[kCtrWork];
  for (;;) {
    if (tid == 0) s_item = atomicAdd(counters + kCtrWorkNext, 1);
    __syncthreads();
    const int item = s_item;
    if (item >= G) break;
    const int4 wk = work[item];
    const int p = wk.x;
    for (int i = tid; i < H * IN; i += kRowsPerItem) sW1[i] = W1[(size_t)p * H * IN + i];
    for (int i = tid; i < H * H; i += kRowsPerItem) sW2[i] = W2[(size_t)p * H * H + i];
    for (int i = tid; i < 4 * H; i += kRowsPerItem) sW3[i] = W3[(size_t)p * 4 * H + i];
    for (int i = tid; i < H; i += kRowsPerItem) { sb1[i] = b1[(size_t)p * H + i]; sb2[i] = b2[(size_t)p * H + i]; }
    if (tid < 4) sb3[tid] = b3[(size_t)p * 4 + tid];
    if (tid < F) { sfa[tid] = freq[tid]; sfa[F + tid] = att[tid]; }
    __syncthreads();
    if (tid < wk.z) {
      const RecIn r = rec_in[wk.y + tid];
      const float v6[6] = {r.rdx, r.rdy, r.rdz, r.dx, r.dy, r.dz};
      float h1[HMAX];
#pragma unroll
      for (int h = 0; h < HMAX; ++h) h1[h] = (h < H) ? sb1[h] : 0.f;
      for (int c = 0; c < 6; ++c) {
        for (int f = 0; f < F; ++f) {
          const float ph = v6[c] * sfa[f] * sfa[F + f];
          const float sn = __sinf(ph), cs = __cosf(ph);
          const int j = c * F + f;
#pragma unroll
          for (int h = 0; h < HMAX; ++h) {
            if (h < H) {
              h1[h] = fmaf(sW1[h * IN + j], sn, h1[h]);
              h1[h] = fmaf(sW1[h * IN + j + half], cs, h1[h]);
            }
          }
        }
      }
      uint32_t m1 = 0u, m2 = 0u;
#pragma unroll
      for (int h = 0; h < HMAX; ++h) {
        if (h < 32 && h1[h] > 0.f) m1 |= 1u << h;
        h1[h] = fmaxf(h1[h], 0.f);
      }
      float o0 = sb3[0], o1 = sb3[1], o2 = sb3[2], o3 = sb3[3];
      for (int q = 0; q < H; ++q) {
        float a = sb2[q];
#pragma unroll
        for (int h = 0; h < HMAX; ++h) if (h < H) a = fmaf(sW2[q * H + h], h1[h], a);
        if (q < 32 && a > 0.f) m2 |= 1u << q;
        a = fmaxf(a, 0.f);
        // layer 3 accumulates over ascending hidden index, which is this loop's order
        o0 = fmaf(sW3[0 * H + q], a, o0); o1 = fmaf(sW3[1 * H + q], a, o1);
        o2 = fmaf(sW3[2 * H + q], a, o2); o3 = fmaf(sW3[3 * H + q], a, o3);
      }
      const float sigma_raw = softplus_fast(o3);
      float4 out;
      out.x = sigmoid_fast(o0); out.y = sigmoid_fast(o1); out.z = sigmoid_fast(o2);
      out.w = (out_mode == kOutAlpha) ? (1.f - __expf(-(sigma_raw * r.decay))) : sigma_raw;
      rec_out[r.slot] = out;
      if (rec_ext) rec_ext[r.slot] = make_float4(sigma_raw, o3, __uint_as_float(m1), __uint_as_float(m2));
    }
    __syncthreads();
  }
}

// The standard network (6 frequencies, hidden 32) with compile-time sizes: W1 sits transposed in shared memory
// ([input][hidden], rows padded to 36 floats so that the staging stores spread over the banks and every row stays
// 16-byte aligned), so the 32 hidden sums of one input take eight 128-bit broadcast loads instead of 32 scalar ones;
// W2 rows are read the same way.  The order of every sum is the one described at the top of this file.
constexpr int kSH = 32, kSF = 6, kSIN = 72, kSRow = 36;
constexpr int kStdSmemFloats = kSIN * kSRow + kSH * kSH + kSH * 4 + kSH + kSH + 4;

__global__ void __launch_bounds__(kRowsPerItem) k_mlp_f32_std(
    const float* __restrict__ W1, const float* __restrict__ b1, const float* __restrict__ W2,
    const float* __restrict__ b2, const float* __restrict__ W3, const float* __restrict__ b3,
    const float* __restrict__ freq, const float* __restrict__ att, const RecIn* __restrict__ rec_in,
    const int4* __restrict__ work, int32_t* __restrict__ counters, float4* __restrict__ rec_out,
    float4* __restrict__ rec_ext, int out_mode, const int32_t* __restrict__ status) {
  extern __shared__ __align__(16) float sW[];
  __shared__ int s_item;
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  float* sW1T = sW;                          // [72][36]
  float* sW2 = sW1T + kSIN * kSRow;          // [32][32]
  float* sW3T = sW2 + kSH * kSH;             // [32][4]
  float* sb1 = sW3T + kSH * 4;
  float* sb2 = sb1 + kSH;
  float* sb3 = sb2 + kSH;
  const int tid = threadIdx.x;
  const int G = counters[kCtrWork];
  float fr[kSF], at[kSF];
#pragma unroll
  for (int f = 0; f < kSF; ++f) { fr[f] = __ldg(freq + f); at[f] = __ldg(att + f); }
  for (;;) {
    if (tid == 0) s_item = atomicAdd(counters + kCtrWorkNext, 1);
    __syncthreads();
    const int item = s_item;
    if (item >= G) break;
    const int4 wk = work[item];
    const int p = wk.x;
    for (int i = tid; i < kSH * kSIN; i += kRowsPerItem) {
      const int h = i / kSIN, j = i - h * kSIN;
      sW1T[j * kSRow + h] = W1[(size_t)p * kSH * kSIN + i];
    }
    for (int i = tid; i < kSH * kSH; i += kRowsPerItem) sW2[i] = W2[(size_t)p * kSH * kSH + i];
    {
      const int c = tid >> 5, q = tid & 31;   // 128 threads = 4 outputs x 32 hidden
      sW3T[q * 4 + c] = W3[(size_t)p * 4 * kSH + c * kSH + q];
    }
    if (tid < kSH) { sb1[tid] = b1[(size_t)p * kSH + tid]; sb2[tid] = b2[(size_t)p * kSH + tid]; }
    if (tid < 4) sb3[tid] = b3[(size_t)p * 4 + tid];
    __syncthreads();
    if (tid < wk.z) {
      const RecIn r = rec_in[wk.y + tid];
      const float v6[6] = {r.rdx, r.rdy, r.rdz, r.dx, r.dy, r.dz};
      float h1[kSH];
#pragma unroll
      for (int k = 0; k < kSH / 4; ++k) {
        const float4 b = reinterpret_cast<const float4*>(sb1)[k];
        h1[4 * k] = b.x; h1[4 * k + 1] = b.y; h1[4 * k + 2] = b.z; h1[4 * k + 3] = b.w;
      }
#pragma unroll
      for (int c = 0; c < 6; ++c) {
#pragma unroll
        for (int f = 0; f < kSF; ++f) {
          const float ph = v6[c] * fr[f] * at[f];
          const float sn = __sinf(ph), cs = __cosf(ph);
          const int j = c * kSF + f;
          const float4* ws = reinterpret_cast<const float4*>(sW1T + j * kSRow);
          const float4* wc = reinterpret_cast<const float4*>(sW1T + (j + kSIN / 2) * kSRow);
#pragma unroll
          for (int k = 0; k < kSH / 4; ++k) {
            const float4 a = ws[k], b = wc[k];
            h1[4 * k] = fmaf(b.x, cs, fmaf(a.x, sn, h1[4 * k]));
            h1[4 * k + 1] = fmaf(b.y, cs, fmaf(a.y, sn, h1[4 * k + 1]));
            h1[4 * k + 2] = fmaf(b.z, cs, fmaf(a.z, sn, h1[4 * k + 2]));
            h1[4 * k + 3] = fmaf(b.w, cs, fmaf(a.w, sn, h1[4 * k + 3]));
          }
        }
      }
      uint32_t m1 = 0u, m2 = 0u;
#pragma unroll
      for (int h = 0; h < kSH; ++h) {
        if (h1[h] > 0.f) m1 |= 1u << h;
        h1[h] = fmaxf(h1[h], 0.f);
      }
      float o0 = sb3[0], o1 = sb3[1], o2 = sb3[2], o3 = sb3[3];
#pragma unroll 4
      for (int q = 0; q < kSH; ++q) {
        float a = sb2[q];
        const float4* row = reinterpret_cast<const float4*>(sW2 + q * kSH);
#pragma unroll
        for (int k = 0; k < kSH / 4; ++k) {
          const float4 w = row[k];
          a = fmaf(w.x, h1[4 * k], a); a = fmaf(w.y, h1[4 * k + 1], a);
          a = fmaf(w.z, h1[4 * k + 2], a); a = fmaf(w.w, h1[4 * k + 3], a);
        }
        if (a > 0.f) m2 |= 1u << q;
        a = fmaxf(a, 0.f);
        const float4 w3 = reinterpret_cast<const float4*>(sW3T)[q];
        o0 = fmaf(w3.x, a, o0); o1 = fmaf(w3.y, a, o1); o2 = fmaf(w3.z, a, o2); o3 = fmaf(w3.w, a, o3);
      }
      const float sigma_raw = softplus_fast(o3);
      float4 out;
      out.x = sigmoid_fast(o0); out.y = sigmoid_fast(o1); out.z = sigmoid_fast(o2);
      out.w = (out_mode == kOutAlpha) ? (1.f - __expf(-(sigma_raw * r.decay))) : sigma_raw;
      rec_out[r.slot] = out;
      if (rec_ext) rec_ext[r.slot] = make_float4(sigma_raw, o3, __uint_as_float(m1), __uint_as_float(m2));
    }
    __syncthreads();
  }
}

int launch_mlp_f32(const mlpsp_scene* sc, const RecIn* rec_in, const int32_t* prim_off, const int4* work,
                   const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                   cudaStream_t st, int grid_cap) {
  const int H = sc->hidden, F = sc->num_freq;
  MLPSP_REQUIRE(H >= 1 && H <= 64 && F >= 1 && F <= 8, MLPSP_E_LIMIT, "FP32 evaluator needs 1<=H<=64, 1<=F<=8");
  MLPSP_REQUIRE(sc->W1 && sc->b1 && sc->W2 && sc->b2 && sc->W3 && sc->b3 && sc->freq && sc->att, MLPSP_E_ARG,
                "FP32 evaluator needs the FP32 weight arrays");
  const int IN = 12 * F;
  const size_t smem = sizeof(float) * (size_t)(H * IN + H + H * H + H + 4 * H + 4 + 2 * F);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = grid_cap > 0 ? std::min(grid_cap, sms * 8) : sms * 8;
  int32_t* ctr = const_cast<int32_t*>(counters);
  LaunchScope scope(kKMlp, 1, st);
  if (H == kSH && F == kSF) {
    k_mlp_f32_std<<<grid, kRowsPerItem, sizeof(float) * kStdSmemFloats, st>>>(
        sc->W1, sc->b1, sc->W2, sc->b2, sc->W3, sc->b3, sc->freq, sc->att, rec_in, work, ctr, rec_out, rec_ext, out_mode,
        status);
  } else if (H <= 32) {
    k_mlp_f32<32><<<grid, kRowsPerItem, smem, st>>>(sc->W1, sc->b1, sc->W2, sc->b2, sc->W3, sc->b3, sc->freq, sc->att,
                                                   F, H, rec_in, prim_off, work, ctr, rec_out, rec_ext, out_mode, status);
  } else {
    k_mlp_f32<64><<<grid, kRowsPerItem, smem, st>>>(sc->W1, sc->b1, sc->W2, sc->b2, sc->W3, sc->b3, sc->freq, sc->att,
                                                   F, H, rec_in, prim_off, work, ctr, rec_out, rec_ext, out_mode, status);
  }
  return cuda_check(cudaGetLastError(), "mlp_f32");
}

}  // namespace mlpsp
