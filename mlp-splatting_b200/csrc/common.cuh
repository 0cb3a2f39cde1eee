// Shared device helpers for the tile-centre render path (sm_100a only).
//
// Arithmetic contract: every float operation that feeds an integer decision (tile overlap, sort
// order, hit / no hit) is written with explicit round-to-nearest intrinsics, so the compiler can
// neither fuse nor reorder it, and det_exp() replaces the hardware exponential.  A CPU that issues
// the same IEEE-754 binary32 operations in the same order reproduces those decisions bit for bit.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/mlpsp.h"

#define MLPSP_SENTINEL_KEY 1e30f
#define MLPSP_TERM 1e-3f

namespace mlpsp {

__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float ffma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }

// exp(x) from IEEE operations only: Cody-Waite reduction by ln2 (hi/lo), degree-5 polynomial with
// the Cephes expf coefficients, exponent assembled from integer bits.  x < -87 -> 0, x > 88 -> inf.
__device__ __forceinline__ float det_exp(float x) {
  if (!(x >= -87.0f)) return (x != x) ? x : 0.0f;
  if (x > 88.0f) return __int_as_float(0x7f800000);
  const float kf = rintf(fmul(x, 1.44269504088896341f));
  float r = ffma(kf, -0.693359375f, x);
  r = ffma(kf, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = ffma(p, r, 1.3981999507e-3f);
  p = ffma(p, r, 8.3334519073e-3f);
  p = ffma(p, r, 4.1665795894e-2f);
  p = ffma(p, r, 1.6666665459e-1f);
  p = ffma(p, r, 5.0000001201e-1f);
  const float r2 = fmul(r, r);
  float y = ffma(p, r2, r);
  y = fadd(y, 1.0f);
  const int k = (int)kf;
  return fmul(y, __int_as_float((k + 127) << 23));
}

struct V3 { float x, y, z; };

// R^T v for unit quaternion (w,x,y,z): v + w t + u x t, t = 2 (u x v), u = -(x,y,z).
// (scannet/cuda/np_tile_kernels.cu:416-435)
__device__ __forceinline__ V3 rot_conj(float qw, float qx, float qy, float qz, V3 v) {
  const float ux = -qx, uy = -qy, uz = -qz;
  const float tx = fmul(2.f, ffma(uy, v.z, -fmul(uz, v.y)));
  const float ty = fmul(2.f, ffma(uz, v.x, -fmul(ux, v.z)));
  const float tz = fmul(2.f, ffma(ux, v.y, -fmul(uy, v.x)));
  V3 r;
  r.x = fadd(ffma(qw, tx, v.x), ffma(uy, tz, -fmul(uz, ty)));
  r.y = fadd(ffma(qw, ty, v.y), ffma(uz, tx, -fmul(ux, tz)));
  r.z = fadd(ffma(qw, tz, v.z), ffma(ux, ty, -fmul(uy, tx)));
  return r;
}

// Packed primitive geometry: 4 x float4 per primitive.
//   g0 = (cx, cy, cz, qw)   g1 = (qx, qy, qz, max_k exp(ls_k))
//   g2 = (m_x, m_y, m_z, 0) with m_k = exp(-2 ls_k)     g3 = (ls_x, ls_y, ls_z, 0)
struct Geom {
  float cx, cy, cz, qw, qx, qy, qz, smax, mx, my, mz;
};

__device__ __forceinline__ Geom load_geom(const float4* __restrict__ geom, int p) {
  const float4 a = __ldg(geom + (size_t)p * 4 + 0);
  const float4 b = __ldg(geom + (size_t)p * 4 + 1);
  const float4 c = __ldg(geom + (size_t)p * 4 + 2);
  Geom g;
  g.cx = a.x; g.cy = a.y; g.cz = a.z; g.qw = a.w;
  g.qx = b.x; g.qy = b.y; g.qz = b.z; g.smax = b.w;
  g.mx = c.x; g.my = c.y; g.mz = c.z;
  return g;
}

__device__ __forceinline__ float ab_terms(const Geom& g, V3 o, V3 d, float& numer) {
  V3 v = { fsub(g.cx, o.x), fsub(g.cy, o.y), fsub(g.cz, o.z) };
  const V3 vl = rot_conj(g.qw, g.qx, g.qy, g.qz, v);
  const V3 dl = rot_conj(g.qw, g.qx, g.qy, g.qz, d);
  const float denom = ffma(fmul(dl.x, dl.x), g.mx, ffma(fmul(dl.y, dl.y), g.my, fmul(fmul(dl.z, dl.z), g.mz)));
  numer = ffma(fmul(dl.x, vl.x), g.mx, ffma(fmul(dl.y, vl.y), g.my, fmul(fmul(dl.z, vl.z), g.mz)));
  return denom;
}

// Tile-centre ordering key (np_tile_kernels.cu:483-518): t* on the tile-centre ray, 1e30 when the
// ray is degenerate for this primitive or t* <= 0.
__device__ __forceinline__ float tile_key(const Geom& g, V3 o, V3 d) {
  float numer;
  const float denom = ab_terms(g, o, d, numer);
  if (denom <= 1e-20f) return MLPSP_SENTINEL_KEY;
  const float t = fdiv(numer, denom);
  return (t > 0.f) ? t : MLPSP_SENTINEL_KEY;
}

// Euclidean depth of the centre along the tile-centre ray: the ordering key of the reference's
// expected-depth kernel (np_tile_kernels.cu:5538-5543).
__device__ __forceinline__ float tile_key_euclid(const Geom& g, V3 o, V3 d) {
  const float vx = fsub(g.cx, o.x), vy = fsub(g.cy, o.y), vz = fsub(g.cz, o.z);
  const float t = ffma(vx, d.x, ffma(vy, d.y, fmul(vz, d.z)));
  return (t > 0.f) ? t : MLPSP_SENTINEL_KEY;
}

struct Hit { float t, dx, dy, dz, qx, qy, qz, decay; };

// Rotated-ellipsoid closest approach (np_tile_kernels.cu:659-711).
__device__ __forceinline__ bool hit_test(const Geom& g, V3 o, V3 d, float thr, Hit& h) {
  float numer;
  const float denom = ab_terms(g, o, d, numer);
  if (denom <= 1e-20f) return false;
  const float t = fdiv(numer, denom);
  if (!(t > 0.f)) return false;
  const float px = ffma(t, d.x, o.x), py = ffma(t, d.y, o.y), pz = ffma(t, d.z, o.z);
  V3 dd = { fsub(g.cx, px), fsub(g.cy, py), fsub(g.cz, pz) };
  const V3 q = rot_conj(g.qw, g.qx, g.qy, g.qz, dd);
  float r2 = fmul(fmul(q.x, q.x), g.mx);
  r2 = ffma(fmul(q.y, q.y), g.my, r2);
  r2 = ffma(fmul(q.z, q.z), g.mz, r2);
  r2 = fmaxf(r2, 0.f);
  const float decay = det_exp(fmul(-0.5f, r2));
  h.t = t; h.dx = dd.x; h.dy = dd.y; h.dz = dd.z; h.qx = q.x; h.qy = q.y; h.qz = q.z; h.decay = decay;
  return decay > thr;
}

// Cheap necessary condition for a hit: the centre's distance to the ray's line must be below the
// bounding radius.  With r^2 = sum q_k^2 m_k >= |c - p|^2 / smax^2 >= perp^2 / smax^2 for every point p
// of the line, decay > thr needs perp^2 < smax^2 * (-2 ln thr).  bound2 carries a 2 % margin, far
// above any rounding error here, so a rejected pair is one the full test also rejects and the
// decisions stay identical to evaluating hit_test everywhere.  NaNs fall through to the full test.
__device__ __forceinline__ bool surely_misses(const Geom& g, V3 o, V3 d, float bound2) {
  const float vx = g.cx - o.x, vy = g.cy - o.y, vz = g.cz - o.z;
  const float te = vx * d.x + vy * d.y + vz * d.z;
  const float wx = vx - te * d.x, wy = vy - te * d.y, wz = vz - te * d.z;
  return (wx * wx + wy * wy + wz * wz) > bound2 * (g.smax * g.smax);
}

__device__ __forceinline__ V3 load3(const float* __restrict__ p, int64_t i) {
  V3 r = { __ldg(p + i * 3), __ldg(p + i * 3 + 1), __ldg(p + i * 3 + 2) };
  return r;
}

// Output activations (np_tile_kernels.cu:75-83); values, not decisions, so hardware exp is fine.
__device__ __forceinline__ float sigmoid_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float softplus_fast(float x) {
  if (x > 20.f) return x;
  if (x < -20.f) return __expf(x);
  return log1pf(__expf(x));
}

// ---- block-wide exclusive scan of one int per thread (blockDim.x <= 1024, multiple of 32) ----
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums /* [32] shared */, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    int w = (lane < nw) ? warp_sums[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int base = (warp > 0) ? warp_sums[warp - 1] : 0;
  total = warp_sums[((blockDim.x + 31) >> 5) - 1];
  __syncthreads();
  return base + inc - v;
}

}  // namespace mlpsp
