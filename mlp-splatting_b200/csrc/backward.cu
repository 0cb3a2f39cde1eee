// The backward side of the record path: reverse compositing over saved records and the per-primitive
// weight gradients of the grouped MLP.
//
// mlpsp_records_reverse computes what primitive_records_reverse_kernel computes (scannet/cuda/primitive_records.cuh:3-49):
// the image adjoints become the adjoint of every record's four pre-activation MLP outputs plus position /
// log-scale / quaternion gradients accumulated per primitive; see "records reverse" below for how the work is split.
//
// mlpsp_grouped_weight_gradients computes what scannet/primitive_gemm.py:101-279 computes with Triton
// (grouped_weight_gradients, FP32 operand mode) and scannet/primitive_csr.py:33-58 states in PyTorch:
// per primitive, with its records' encoded inputs E, saved ReLU masks and output adjoints D3,
//   D2 = (D3 W3) * mask2,  D1 = (D2 W2) * mask1,
//   dW3 = D3^T H2, db3 = sum D3, dW2 = D2^T H1, db2 = sum D2, dW1 = D1^T E, db1 = sum D1.
// One CTA handles one prepared segment of one primitive in blocks of 128 records (thread = record for the
// forward recomputation and the adjoints, then thread = output element for the D^T X products over the block
// in shared memory) and writes a partial 3,524-vector; a second kernel adds a primitive's partials in segment
// order, so the result does not depend on scheduling, and raises the non-finite flag.
#include "frame.cuh"

namespace mlpsp {

// ------------------------------------------------------------------ quaternion helpers ----
// rotate v by the unit quaternion (w, x, y, z): v + w t + u x t with t = 2 (u x v), u = (x, y, z)
__device__ __forceinline__ V3 rot_quat(float qw, float qx, float qy, float qz, V3 v) {
  const float tx = 2.f * (qy * v.z - qz * v.y), ty = 2.f * (qz * v.x - qx * v.z), tz = 2.f * (qx * v.y - qy * v.x);
  V3 r;
  r.x = v.x + qw * tx + (qy * tz - qz * ty);
  r.y = v.y + qw * ty + (qz * tx - qx * tz);
  r.z = v.z + qw * tz + (qx * ty - qy * tx);
  return r;
}

// Chain rule from the adjoint G of the rotation matrix R(q) (row-major 3x3) to the quaternion
// (np_tile_kernels.cu:439-480).  With R = I + 2 w [u]x + 2 [u]x^2 the partial derivatives are
//   dR/dw = 2 [u]x,   dR/du_k = 2 w [e_k]x + 2 ([e_k]x [u]x + [u]x [e_k]x).
__device__ __forceinline__ void quat_adjoint(float w, float x, float y, float z, const float (&G)[9], float (&gq)[4]) {
  const float u[3] = {x, y, z};
  // [a]x as a row-major matrix
  auto cross_m = [](const float a[3], float M[9]) {
    M[0] = 0.f;   M[1] = -a[2]; M[2] = a[1];
    M[3] = a[2];  M[4] = 0.f;   M[5] = -a[0];
    M[6] = -a[1]; M[7] = a[0];  M[8] = 0.f;
  };
  float U[9];
  cross_m(u, U);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 9; ++i) acc += G[i] * 2.f * U[i];
  gq[0] = acc;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    float e[3] = {0.f, 0.f, 0.f};
    e[k] = 1.f;
    float E[9];
    cross_m(e, E);
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        float eu = 0.f, ue = 0.f;
#pragma unroll
        for (int m = 0; m < 3; ++m) { eu += E[r * 3 + m] * U[m * 3 + c]; ue += U[r * 3 + m] * E[m * 3 + c]; }
        s += G[r * 3 + c] * (2.f * w * E[r * 3 + c] + 2.f * (eu + ue));
      }
    gq[1 + k] = s;
  }
}

// ------------------------------------------------------------------- records reverse ----
// The reference walks a pixel's records backwards in one thread and issues ten (warp-aggregated) global atomics per
// record from inside that walk (primitive_records.cuh:3-49).  Here the walk is reduced to what is sequential -- the
// recurrence of the colour that lies behind a record -- and everything else runs record-parallel afterwards:
//   k_reverse_pixels    thread = pixel: the recurrence, the three colour adjoints of every record, and
//                       g_sigma * decay parked in the fourth adjoint;
//   k_reverse_geometry  thread = record: the opacity adjoint is finished, the position / log-scale / quaternion
//                       contributions are computed and summed per primitive in a shared-memory table first (records
//                       that follow one another belong to neighbouring pixels, which mostly see the same
//                       primitives), so that global memory sees one set of atomics per primitive and chunk of
//                       records instead of one per record.
__global__ void k_reverse_pixels(const int64_t* __restrict__ offsets, const float* __restrict__ raw,
                                 const float* __restrict__ grgb, const float* __restrict__ gt, int64_t pixels,
                                 float* __restrict__ d4) {
  const int64_t pix = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (pix >= pixels) return;
  const float gr = grgb[pix * 3], gg = grgb[pix * 3 + 1], gb = grgb[pix * 3 + 2];
  float behind = gt[pix];   // adjoint of the transmittance that reaches whatever lies behind the current record
  for (int64_t r = offsets[pix + 1] - 1; r >= offsets[pix]; --r) {
    const float4 a = *reinterpret_cast<const float4*>(raw + r * 8);        // R, G, B, sigma_raw
    const float4 c = *reinterpret_cast<const float4*>(raw + r * 8 + 4);    // trans before, alpha, decay, sigma logit
    const float colour = gr * a.x + gg * a.y + gb * a.z;
    const float g_alpha = c.x * (colour - behind);
    behind = behind * (1.f - c.y) + colour * c.y;
    const float g_sigma = g_alpha * __expf(-a.w * c.z);   // d alpha / d (sigma_raw * decay) = 1 - alpha
    const float w = c.x * c.y;
    *reinterpret_cast<float4*>(d4 + r * 4) = make_float4(gr * w * a.x * (1.f - a.x), gg * w * a.y * (1.f - a.y),
                                                         gb * w * a.z * (1.f - a.z), g_sigma * c.z);
  }
}

constexpr int kRevThreads = 256;
constexpr int kRevChunk = 4096;      // records per CTA
constexpr int kRevTable = 1024;      // shared-memory accumulator rows (a power of two)
constexpr int kRevProbe = 16;        // probes before a record goes to global memory directly

__global__ void __launch_bounds__(kRevThreads) k_reverse_geometry(
    const int32_t* __restrict__ ids, const float* __restrict__ x6, const float* __restrict__ raw,
    const float* __restrict__ logs, const float* __restrict__ quats, int64_t total, float* __restrict__ d4,
    float* __restrict__ gp, float* __restrict__ gs, float* __restrict__ gq) {
  __shared__ int s_key[kRevTable];
  __shared__ float s_acc[kRevTable][10];
  for (int i = threadIdx.x; i < kRevTable; i += kRevThreads) {
    s_key[i] = -1;
#pragma unroll
    for (int j = 0; j < 10; ++j) s_acc[i][j] = 0.f;
  }
  __syncthreads();
  const int64_t r0 = (int64_t)blockIdx.x * kRevChunk;
  const int64_t r1 = r0 + kRevChunk < total ? r0 + kRevChunk : total;
  for (int64_t r = r0 + threadIdx.x; r < r1; r += kRevThreads) {
    const int p = ids[r];
    const float4 a = *reinterpret_cast<const float4*>(raw + r * 8);        // .w = sigma_raw
    const float4 c = *reinterpret_cast<const float4*>(raw + r * 8 + 4);    // .z = decay, .w = sigma logit
    const float parked = d4[r * 4 + 3];                                    // g_sigma * decay
    d4[r * 4 + 3] = parked * sigmoid_fast(c.w);                            // softplus' = sigmoid
    // decay = exp(-1/2 q^T M q), q = R^T d, d = c - foot point (x6[3..5]), M = diag(exp(-2 ls))
    const float k = parked * a.w;                                          // g_decay * decay = g_sigma * sigma_raw * decay
    const V3 d = {x6[r * 6 + 3], x6[r * 6 + 4], x6[r * 6 + 5]};
    const float4 qt = *reinterpret_cast<const float4*>(quats + (size_t)p * 4);
    const V3 q = rot_conj_fast(qt.x, qt.y, qt.z, qt.w, d);
    const float mx = __expf(-2.f * logs[p * 3]), my = __expf(-2.f * logs[p * 3 + 1]), mz = __expf(-2.f * logs[p * 3 + 2]);
    const V3 gl = {-k * mx * q.x, -k * my * q.y, -k * mz * q.z};           // adjoint of q
    const V3 gd = rot_quat(qt.x, qt.y, qt.z, qt.w, gl);                    // adjoint of d, hence of the centre
    // q = R^T d  =>  adjoint of R is d gl^T
    const float Gm[9] = {d.x * gl.x, d.x * gl.y, d.x * gl.z, d.y * gl.x, d.y * gl.y, d.y * gl.z,
                         d.z * gl.x, d.z * gl.y, d.z * gl.z};
    float gquat[4];
    quat_adjoint(qt.x, qt.y, qt.z, qt.w, Gm, gquat);
    const float v[10] = {gd.x, gd.y, gd.z, k * mx * q.x * q.x, k * my * q.y * q.y, k * mz * q.z * q.z,
                         gquat[0], gquat[1], gquat[2], gquat[3]};
    // the primitive's row of the table: linear probing from a multiplicative hash
    int slot = (int)(((uint32_t)p * 2654435761u) >> 22) & (kRevTable - 1);
    bool placed = false;
    for (int probe = 0; probe < kRevProbe && !placed; ++probe) {
      const int seen = atomicCAS(&s_key[slot], -1, p);
      if (seen == -1 || seen == p) placed = true;
      else slot = (slot + 1) & (kRevTable - 1);
    }
    if (placed) {
#pragma unroll
      for (int j = 0; j < 10; ++j) atomicAdd(&s_acc[slot][j], v[j]);
    } else {
      atomicAdd(gp + p * 3, v[0]); atomicAdd(gp + p * 3 + 1, v[1]); atomicAdd(gp + p * 3 + 2, v[2]);
      atomicAdd(gs + p * 3, v[3]); atomicAdd(gs + p * 3 + 1, v[4]); atomicAdd(gs + p * 3 + 2, v[5]);
      atomicAdd(gq + p * 4, v[6]); atomicAdd(gq + p * 4 + 1, v[7]); atomicAdd(gq + p * 4 + 2, v[8]); atomicAdd(gq + p * 4 + 3, v[9]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kRevTable; i += kRevThreads) {
    const int p = s_key[i];
    if (p < 0) continue;
    atomicAdd(gp + p * 3, s_acc[i][0]); atomicAdd(gp + p * 3 + 1, s_acc[i][1]); atomicAdd(gp + p * 3 + 2, s_acc[i][2]);
    atomicAdd(gs + p * 3, s_acc[i][3]); atomicAdd(gs + p * 3 + 1, s_acc[i][4]); atomicAdd(gs + p * 3 + 2, s_acc[i][5]);
    atomicAdd(gq + p * 4, s_acc[i][6]); atomicAdd(gq + p * 4 + 1, s_acc[i][7]);
    atomicAdd(gq + p * 4 + 2, s_acc[i][8]); atomicAdd(gq + p * 4 + 3, s_acc[i][9]);
  }
}

// --------------------------------------------------------- grouped weight gradients ----
constexpr int kGH = 32, kGIN = 72, kGSeg = 128;
constexpr int kOW1 = 0, kOb1 = kOW1 + kGH * kGIN, kOW2 = kOb1 + kGH, kOb2 = kOW2 + kGH * kGH, kOW3 = kOb2 + kGH,
              kOb3 = kOW3 + 4 * kGH, kGradLen = kOb3 + 4;   // 3,524 = the reference's packed gradient row
static_assert(kGradLen == 3524, "gradient row layout");

// shared memory: weights of the primitive, then per record E[72], H1[32], H2[32], D1[32], D2[32], D3[4]
constexpr int kRowF = kGIN + 4 * kGH + 4;                       // 204 floats per record
constexpr int kGradSmem = (kGH * kGIN + kGH * kGH + 4 * kGH + 2 * kGH) * 4 + kGSeg * kRowF * 4;

constexpr int kOutPerThread = (kGradLen + kGSeg - 1) / kGSeg;   // 28

__global__ void __launch_bounds__(kGSeg) k_grouped_vjp(
    const float* __restrict__ x6, const float* __restrict__ d4, const int32_t* __restrict__ masks,
    const int64_t* __restrict__ offsets, const int64_t* __restrict__ seg_prim, const int64_t* __restrict__ seg_start,
    int segment_size, const float* __restrict__ freq, const float* __restrict__ att, const float* __restrict__ W1,
    const float* __restrict__ b1, const float* __restrict__ W2, const float* __restrict__ b2,
    const float* __restrict__ W3, float scale, float* __restrict__ partial) {
  extern __shared__ float sm[];
  float* sW1 = sm;
  float* sW2 = sW1 + kGH * kGIN;
  float* sW3 = sW2 + kGH * kGH;
  float* sb1 = sW3 + 4 * kGH;
  float* sb2 = sb1 + kGH;
  float* rows = sb2 + kGH;
  const int seg = blockIdx.x, tid = threadIdx.x;
  const int p = (int)seg_prim[seg];
  const int64_t begin = seg_start[seg];
  const int total = (int)min((int64_t)segment_size, offsets[p + 1] - begin);
  for (int i = tid; i < kGH * kGIN; i += kGSeg) sW1[i] = W1[(size_t)p * kGH * kGIN + i];
  for (int i = tid; i < kGH * kGH; i += kGSeg) sW2[i] = W2[(size_t)p * kGH * kGH + i];
  for (int i = tid; i < 4 * kGH; i += kGSeg) sW3[i] = W3[(size_t)p * 4 * kGH + i];
  if (tid < kGH) { sb1[tid] = b1[(size_t)p * kGH + tid]; sb2[tid] = b2[(size_t)p * kGH + tid]; }
  float acc[kOutPerThread];
#pragma unroll
  for (int k = 0; k < kOutPerThread; ++k) acc[k] = 0.f;
  float* me = rows + (size_t)tid * kRowF;
  float* E = me, *H1 = me + kGIN, *H2 = H1 + kGH, *D1 = H2 + kGH, *D2 = D1 + kGH, *D3 = D2 + kGH;
  for (int sub = 0; sub < total; sub += kGSeg) {
    const int cnt = min(kGSeg, total - sub);
    __syncthreads();   // weights loaded / the previous block's rows consumed
    if (tid < cnt) {
      const int64_t r = begin + sub + tid;
      // encoding as scannet/cumodel.py:183-195: index c*F + f holds sin, + 36 holds cos
      for (int c = 0; c < 6; ++c) {
        const float v = x6[r * 6 + c];
        for (int f = 0; f < 6; ++f) {
          const float ph = v * freq[f] * att[f];
          E[c * 6 + f] = sinf(ph);
          E[36 + c * 6 + f] = cosf(ph);
        }
      }
      uint32_t m1 = 0, m2 = 0;
      if (masks) { m1 = (uint32_t)masks[r * 2]; m2 = (uint32_t)masks[r * 2 + 1]; }
      for (int h = 0; h < kGH; ++h) {
        float a = sb1[h];
        for (int j = 0; j < kGIN; ++j) a = fmaf(sW1[h * kGIN + j], E[j], a);
        if (!masks && a > 0.f) m1 |= 1u << h;
        H1[h] = a > 0.f ? a : 0.f;
      }
      for (int q = 0; q < kGH; ++q) {
        float a = sb2[q];
        for (int h = 0; h < kGH; ++h) a = fmaf(sW2[q * kGH + h], H1[h], a);
        if (!masks && a > 0.f) m2 |= 1u << q;
        H2[q] = a > 0.f ? a : 0.f;
      }
      for (int c = 0; c < 4; ++c) D3[c] = d4[r * 4 + c] * scale;
      for (int h = 0; h < kGH; ++h) {
        float a = 0.f;
        for (int c = 0; c < 4; ++c) a = fmaf(D3[c], sW3[c * kGH + h], a);
        D2[h] = ((m2 >> h) & 1u) ? a : 0.f;
      }
      for (int h = 0; h < kGH; ++h) {
        float a = 0.f;
        for (int q = 0; q < kGH; ++q) a = fmaf(D2[q], sW2[q * kGH + h], a);
        D1[h] = ((m1 >> h) & 1u) ? a : 0.f;
      }
    }
    __syncthreads();
    // thread = output element: sums over the block's records in record order
#pragma unroll
    for (int k = 0; k < kOutPerThread; ++k) {
      const int o = tid + k * kGSeg;
      if (o >= kGradLen) break;
      int a_off, b_off;   // offsets of the two factors inside a record's row; b_off < 0: plain sum of the first
      if (o < kOb1) { a_off = kGIN + 2 * kGH + (o / kGIN); b_off = o % kGIN; }                                   // D1[h] * E[j]
      else if (o < kOW2) { a_off = kGIN + 2 * kGH + (o - kOb1); b_off = -1; }                                    // sum D1[h]
      else if (o < kOb2) { const int e = o - kOW2; a_off = kGIN + 3 * kGH + e / kGH; b_off = kGIN + e % kGH; }   // D2[q] * H1[h]
      else if (o < kOW3) { a_off = kGIN + 3 * kGH + (o - kOb2); b_off = -1; }                                    // sum D2[q]
      else if (o < kOb3) { const int e = o - kOW3; a_off = kGIN + 4 * kGH + e / kGH; b_off = kGIN + kGH + e % kGH; }  // D3[c] * H2[h]
      else { a_off = kGIN + 4 * kGH + (o - kOb3); b_off = -1; }                                                  // sum D3[c]
      float a = acc[k];
      if (b_off >= 0) for (int r = 0; r < cnt; ++r) a = fmaf(rows[(size_t)r * kRowF + a_off], rows[(size_t)r * kRowF + b_off], a);
      else for (int r = 0; r < cnt; ++r) a += rows[(size_t)r * kRowF + a_off];
      acc[k] = a;
    }
  }
  float* out = partial + (size_t)seg * kGradLen;
  const float inv = 1.f / scale;
#pragma unroll
  for (int k = 0; k < kOutPerThread; ++k) {
    const int o = tid + k * kGSeg;
    if (o < kGradLen) out[o] = acc[k] * inv;
  }
}

// result[p] = sum of the partial rows of p's segments, in segment order; nonfinite |= any non-finite sum
__global__ void k_reduce_partials(const float* __restrict__ partial, const int64_t* __restrict__ seg_offsets, int n,
                                  float* __restrict__ result, int32_t* __restrict__ nonfinite) {
  const int p = blockIdx.x;
  const int o = blockIdx.y * blockDim.x + threadIdx.x;
  if (p >= n || o >= kGradLen) return;
  float acc = 0.f;
  for (int64_t g = seg_offsets[p]; g < seg_offsets[p + 1]; ++g) acc += partial[(size_t)g * kGradLen + o];
  result[(size_t)p * kGradLen + o] = acc;
  if (!(fabsf(acc) <= 3.4028235e38f)) atomicOr(nonfinite, 1);
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int mlpsp_records_reverse(const int32_t* ids, const int64_t* offsets, const float* x6, const float* raw,
                                     const float* log_scales, const float* quats, const float* grad_rgb,
                                     const float* grad_t, int64_t pixels, int64_t total_records, int32_t n, float* d4,
                                     float* grad_pos, float* grad_log_scales, float* grad_quats, void* stream) {
  MLPSP_REQUIRE(pixels >= 0 && n >= 0, MLPSP_E_ARG, "mlpsp_records_reverse: negative size");
  MLPSP_REQUIRE(offsets && grad_pos && grad_log_scales && grad_quats, MLPSP_E_ARG, "mlpsp_records_reverse: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  MLPSP_CUDA_OK(cudaMemsetAsync(grad_pos, 0, sizeof(float) * 3 * (size_t)n, st));
  MLPSP_CUDA_OK(cudaMemsetAsync(grad_log_scales, 0, sizeof(float) * 3 * (size_t)n, st));
  MLPSP_CUDA_OK(cudaMemsetAsync(grad_quats, 0, sizeof(float) * 4 * (size_t)n, st));
  if (pixels == 0) return MLPSP_OK;
  MLPSP_REQUIRE(ids && x6 && raw && log_scales && quats && grad_rgb && grad_t && d4, MLPSP_E_ARG,
                "mlpsp_records_reverse: null pointer");
  MLPSP_REQUIRE(total_records >= 0, MLPSP_E_ARG, "mlpsp_records_reverse: negative record count");
  MLPSP_REQUIRE((reinterpret_cast<uintptr_t>(raw) & 15) == 0 && (reinterpret_cast<uintptr_t>(d4) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(quats) & 15) == 0, MLPSP_E_ARG,
                "mlpsp_records_reverse: raw, d4 and quats must be 16-byte aligned");
  LaunchScope scope(kKMisc, 2, st);
  k_reverse_pixels<<<(unsigned)((pixels + 127) / 128), 128, 0, st>>>(offsets, raw, grad_rgb, grad_t, pixels, d4);
  if (total_records > 0)
    k_reverse_geometry<<<(unsigned)((total_records + kRevChunk - 1) / kRevChunk), kRevThreads, 0, st>>>(
        ids, x6, raw, log_scales, quats, total_records, d4, grad_pos, grad_log_scales, grad_quats);
  return cuda_check(cudaGetLastError(), "records_reverse");
}

extern "C" int64_t mlpsp_grouped_gradient_floats(void) { return kGradLen; }

extern "C" int mlpsp_grouped_weight_gradients(const mlpsp_scene* sc, const int64_t* offsets, const float* x6,
                                              const float* d4, const int32_t* relu_masks, const int64_t* seg_prim,
                                              const int64_t* seg_start, const int64_t* seg_offsets, int64_t num_segments,
                                              int32_t segment_size, int32_t precision, float loss_scale, float* partial,
                                              float* result, int32_t* nonfinite, void* stream) {
  MLPSP_REQUIRE(sc && offsets && result && nonfinite, MLPSP_E_ARG, "mlpsp_grouped_weight_gradients: null pointer");
  MLPSP_REQUIRE(sc->hidden == kGH && sc->num_freq == 6, MLPSP_E_LIMIT,
                "grouped backward requires the 72->32->32->4 architecture");
  MLPSP_REQUIRE(sc->W1 && sc->b1 && sc->W2 && sc->b2 && sc->W3 && sc->freq && sc->att, MLPSP_E_ARG,
                "mlpsp_grouped_weight_gradients: FP32 weights missing");
  MLPSP_REQUIRE(loss_scale > 0.f && num_segments >= 0 && num_segments < (1ll << 31) && segment_size > 0, MLPSP_E_ARG,
                "mlpsp_grouped_weight_gradients: bad loss scale, segment size or segment count");
  MLPSP_REQUIRE(precision == MLPSP_PRECISION_F32 || precision == MLPSP_PRECISION_F16 || precision == MLPSP_PRECISION_BF16,
                MLPSP_E_ARG, "mlpsp_grouped_weight_gradients: unsupported operand precision %d", precision);
  // every pointer a launch below reads is checked before the first CUDA call
  MLPSP_REQUIRE(sc->n == 0 || num_segments == 0 || (x6 && d4 && seg_prim && seg_start && seg_offsets && partial),
                MLPSP_E_ARG, "mlpsp_grouped_weight_gradients: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  MLPSP_CUDA_OK(cudaMemsetAsync(nonfinite, 0, 4, st));
  if (sc->n == 0) return MLPSP_OK;
  if (num_segments == 0) {
    // no records at all: every primitive's gradient row is zero
    return cuda_check(cudaMemsetAsync(result, 0, sizeof(float) * (size_t)sc->n * kGradLen, st), "grouped_weight_gradients");
  }
  LaunchScope scope(kKMisc, 2, st);
  if (precision != MLPSP_PRECISION_F32) {
    // binary16 / bfloat16 operands on the tensor cores, FP32 accumulation over the segment
    MLPSP_REQUIRE((reinterpret_cast<uintptr_t>(d4) & 15) == 0, MLPSP_E_ARG,
                  "mlpsp_grouped_weight_gradients: d4 must be 16-byte aligned");
    const int rc = launch_grouped_vjp_tc(precision == MLPSP_PRECISION_BF16, x6, d4, relu_masks, offsets, seg_prim, seg_start,
                                         num_segments, segment_size, sc, loss_scale, partial, nonfinite, st);
    if (rc) return rc;
    const dim3 grid_r(sc->n, (kGradLen + 255) / 256);
    k_reduce_partials<<<grid_r, 256, 0, st>>>(partial, seg_offsets, sc->n, result, nonfinite);
    return cuda_check(cudaGetLastError(), "grouped_weight_gradients");
  }
  static DeviceOnce attr_once;
  if (attr_once.first())
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_grouped_vjp, cudaFuncAttributeMaxDynamicSharedMemorySize, kGradSmem));
  k_grouped_vjp<<<(unsigned)num_segments, kGSeg, kGradSmem, st>>>(x6, d4, relu_masks, offsets, seg_prim, seg_start, segment_size,
                                                                  sc->freq, sc->att, sc->W1, sc->b1, sc->W2, sc->b2, sc->W3,
                                                                  loss_scale, partial);
  const dim3 grid(sc->n, (kGradLen + 255) / 256);
  k_reduce_partials<<<grid, 256, 0, st>>>(partial, seg_offsets, sc->n, result, nonfinite);
  return cuda_check(cudaGetLastError(), "grouped_weight_gradients");
}
