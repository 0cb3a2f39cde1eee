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

// ab_terms with the local-frame offset vl = R^T (c - o) supplied by the caller: for rays that share one origin it
// is the same three numbers for every ray, bit for bit, whichever thread computes them.
__device__ __forceinline__ float ab_terms_vl(const Geom& g, V3 vl, V3 d, float& numer) {
  const V3 dl = rot_conj(g.qw, g.qx, g.qy, g.qz, d);
  const float denom = ffma(fmul(dl.x, dl.x), g.mx, ffma(fmul(dl.y, dl.y), g.my, fmul(fmul(dl.z, dl.z), g.mz)));
  numer = ffma(fmul(dl.x, vl.x), g.mx, ffma(fmul(dl.y, vl.y), g.my, fmul(fmul(dl.z, vl.z), g.mz)));
  return denom;
}
__device__ __forceinline__ V3 local_offset(const Geom& g, V3 o) {
  V3 v = { fsub(g.cx, o.x), fsub(g.cy, o.y), fsub(g.cz, o.z) };
  return rot_conj(g.qw, g.qx, g.qy, g.qz, v);
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

// Rotated-ellipsoid closest approach (np_tile_kernels.cu:659-711).  HAVE_VL: vl = local_offset(g, o) comes from
// the caller (same operations, same bits).
template <bool HAVE_VL>
__device__ __forceinline__ bool hit_test_t(const Geom& g, V3 o, V3 d, V3 vl, float thr, Hit& h) {
  float numer;
  const float denom = HAVE_VL ? ab_terms_vl(g, vl, d, numer) : ab_terms(g, o, d, numer);
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
__device__ __forceinline__ bool hit_test(const Geom& g, V3 o, V3 d, float thr, Hit& h) {
  return hit_test_t<false>(g, o, d, V3{0.f, 0.f, 0.f}, thr, h);
}

// The same geometry for a pair that is already known to hit: t, the offset c - p, its local-frame image
// and decay as plain float values for the evaluator and the compositor.  No decision hangs on them, so
// the compiler may fuse and the hardware reciprocal / exponential are used.
__device__ __forceinline__ V3 rot_conj_fast(float qw, float qx, float qy, float qz, V3 v) {
  const float tx = 2.f * (qz * v.y - qy * v.z), ty = 2.f * (qx * v.z - qz * v.x), tz = 2.f * (qy * v.x - qx * v.y);
  V3 r;
  r.x = v.x + qw * tx + (qz * ty - qy * tz);
  r.y = v.y + qw * ty + (qx * tz - qz * tx);
  r.z = v.z + qw * tz + (qy * tx - qx * ty);
  return r;
}

__device__ __forceinline__ void hit_values_fast(const Geom& g, V3 o, V3 d, Hit& h) {
  const V3 v = {g.cx - o.x, g.cy - o.y, g.cz - o.z};
  const V3 vl = rot_conj_fast(g.qw, g.qx, g.qy, g.qz, v);
  const V3 dl = rot_conj_fast(g.qw, g.qx, g.qy, g.qz, d);
  const float denom = dl.x * dl.x * g.mx + dl.y * dl.y * g.my + dl.z * dl.z * g.mz;
  const float numer = dl.x * vl.x * g.mx + dl.y * vl.y * g.my + dl.z * vl.z * g.mz;
  const float t = __fdividef(numer, denom);
  const V3 dd = {g.cx - (o.x + t * d.x), g.cy - (o.y + t * d.y), g.cz - (o.z + t * d.z)};
  const V3 q = rot_conj_fast(g.qw, g.qx, g.qy, g.qz, dd);
  const float r2 = fmaxf(q.x * q.x * g.mx + q.y * q.y * g.my + q.z * q.z * g.mz, 0.f);
  h.t = t; h.dx = dd.x; h.dy = dd.y; h.dz = dd.z; h.qx = q.x; h.qy = q.y; h.qz = q.z;
  h.decay = __expf(-0.5f * r2);
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

// ---- the reference kernels' own arithmetic (frame.hit_arith = 1) ----
// The decisions above use IEEE-only operations so that a CPU can reproduce them bit for bit.  The reference's
// kernels evaluate the same formulas with the hardware exponential and leave the contraction of a * b + c to the
// compiler (np_tile_kernels.cu:416-435 rotation, 483-518 tile-centre key, 659-711 hit test).  The functions below
// state the formulas in that form -- plain float expressions in the reference's association, fmaf only where the
// reference writes fmaf, __expf where it writes __expf, compiled by the same compiler with the same default
// contraction -- so that on the GPU the keys, the hit decisions and the hit values come out as the reference
// kernels' own do.  No CPU reproduces those bits; CPU checks of this mode need a margin around the threshold.
struct GeomRef { float cx, cy, cz, qw, qx, qy, qz, lsx, lsy, lsz; };

__device__ __forceinline__ GeomRef load_geom_ref(const float4* __restrict__ geom, int p) {
  const float4 a = __ldg(geom + (size_t)p * 4 + 0);
  const float4 b = __ldg(geom + (size_t)p * 4 + 1);
  const float4 c = __ldg(geom + (size_t)p * 4 + 3);
  GeomRef g;
  g.cx = a.x; g.cy = a.y; g.cz = a.z; g.qw = a.w;
  g.qx = b.x; g.qy = b.y; g.qz = b.z;
  g.lsx = c.x; g.lsy = c.y; g.lsz = c.z;
  return g;
}

// v + w t + u x t with t = 2 (u x v), u = (x, y, z); the conjugate rotation passes -u
__device__ __forceinline__ V3 rot_ref(float w, float x, float y, float z, V3 v) {
  const float tx = 2.f * (y * v.z - z * v.y);
  const float ty = 2.f * (z * v.x - x * v.z);
  const float tz = 2.f * (x * v.y - y * v.x);
  V3 r;
  r.x = v.x + w * tx + (y * tz - z * ty);
  r.y = v.y + w * ty + (z * tx - x * tz);
  r.z = v.z + w * tz + (x * ty - y * tx);
  return r;
}

__device__ __forceinline__ float tile_key_ref(const GeomRef& g, V3 o, V3 d) {
  const float vx = g.cx - o.x, vy = g.cy - o.y, vz = g.cz - o.z;
  const float mx = __expf(-2.f * g.lsx), my = __expf(-2.f * g.lsy), mz = __expf(-2.f * g.lsz);
  const V3 vl = rot_ref(g.qw, -g.qx, -g.qy, -g.qz, V3{vx, vy, vz});
  const V3 dl = rot_ref(g.qw, -g.qx, -g.qy, -g.qz, d);
  const float denom = fmaf(dl.x * dl.x, mx, fmaf(dl.y * dl.y, my, (dl.z * dl.z) * mz));
  const float numer = fmaf(dl.x * vl.x, mx, fmaf(dl.y * vl.y, my, (dl.z * vl.z) * mz));
  if (denom <= 1e-20f) return MLPSP_SENTINEL_KEY;
  const float t = numer / denom;
  return (t > 0.f) ? t : MLPSP_SENTINEL_KEY;
}

__device__ __forceinline__ bool hit_test_ref(const GeomRef& g, V3 o, V3 d, float thr, Hit& h) {
  const float vx = g.cx - o.x, vy = g.cy - o.y, vz = g.cz - o.z;
  const float mx = __expf(-2.f * g.lsx), my = __expf(-2.f * g.lsy), mz = __expf(-2.f * g.lsz);
  const V3 vl = rot_ref(g.qw, -g.qx, -g.qy, -g.qz, V3{vx, vy, vz});
  const V3 dl = rot_ref(g.qw, -g.qx, -g.qy, -g.qz, d);
  const float denom = fmaf(dl.x * dl.x, mx, fmaf(dl.y * dl.y, my, (dl.z * dl.z) * mz));
  if (denom <= 1e-20f) return false;
  const float numer = fmaf(dl.x * vl.x, mx, fmaf(dl.y * vl.y, my, (dl.z * vl.z) * mz));
  const float t = numer / denom;
  if (t <= 0.f) return false;
  const float px = o.x + t * d.x, py = o.y + t * d.y, pz = o.z + t * d.z;
  const float dx = g.cx - px, dy = g.cy - py, dz = g.cz - pz;
  const V3 q = rot_ref(g.qw, -g.qx, -g.qy, -g.qz, V3{dx, dy, dz});
  const float r2 = fmaxf(q.x * q.x * mx + q.y * q.y * my + q.z * q.z * mz, 0.f);
  const float decay = __expf(-0.5f * r2);
  h.t = t; h.dx = dx; h.dy = dy; h.dz = dz; h.qx = q.x; h.qy = q.y; h.qz = q.z; h.decay = decay;
  return decay > thr;
}

// ---- per-tile ray frame and the (tile, primitive) pre-test of the fused frame path ----
// All rays of a tile leave one origin o; with an orthonormal frame (a, u, v), a along the tile's mean
// direction, every ray direction is a + alpha u + beta v up to scale (alpha = d.u / d.a, beta = d.v / d.a),
// and the tile's 64 rays lie inside the rectangle [a0, a1] x [b0, b1] of those coordinates (slightly
// inflated).  a0 > a1 marks a tile without such a frame (several origins, a ray more than 60 degrees off the
// mean, non-finite input): no candidate of it is ever rejected.
struct __align__(16) TileFrame {
  float ox, oy, oz, a0;
  float ax, ay, az, a1;
  float ux, uy, uz, b0;
  float vx, vy, vz, b1;
};

__device__ __forceinline__ float quad_min_1d(float A, float B, float C, float lo, float hi) {
  // min over [lo, hi] of A t^2 + 2 B t + C
  const float qlo = fmaf(fmaf(A, lo, 2.f * B), lo, C), qhi = fmaf(fmaf(A, hi, 2.f * B), hi, C);
  float m = fminf(qlo, qhi);
  if (A > 0.f) {
    const float t = fminf(fmaxf(__fdividef(-B, A), lo), hi);
    m = fminf(m, fmaf(fmaf(A, t, 2.f * B), t, C));
  }
  return m;
}

// Whitening map of one primitive: x -> diag(1 / exp(ls)) R^T x as a 3x3 matrix (row-major), its centre, the
// largest inverse scale.  Built once per primitive, used for every tile of its rectangle.
struct PrimWhiten { float m[9]; float cx, cy, cz, ismax; };

__device__ __forceinline__ PrimWhiten make_whiten(const Geom& g) {
  PrimWhiten w;
  const float is[3] = {sqrtf(g.mx), sqrtf(g.my), sqrtf(g.mz)};
  const V3 c0 = rot_conj(g.qw, g.qx, g.qy, g.qz, V3{1.f, 0.f, 0.f});
  const V3 c1 = rot_conj(g.qw, g.qx, g.qy, g.qz, V3{0.f, 1.f, 0.f});
  const V3 c2 = rot_conj(g.qw, g.qx, g.qy, g.qz, V3{0.f, 0.f, 1.f});
  w.m[0] = c0.x * is[0]; w.m[1] = c1.x * is[0]; w.m[2] = c2.x * is[0];
  w.m[3] = c0.y * is[1]; w.m[4] = c1.y * is[1]; w.m[5] = c2.y * is[1];
  w.m[6] = c0.z * is[2]; w.m[7] = c1.z * is[2]; w.m[8] = c2.z * is[2];
  w.cx = g.cx; w.cy = g.cy; w.cz = g.cz;
  w.ismax = fmaxf(is[0], fmaxf(is[1], is[2]));
  return w;
}

__device__ __forceinline__ V3 whiten(const PrimWhiten& w, float x, float y, float z) {
  V3 r;
  r.x = fmaf(w.m[0], x, fmaf(w.m[1], y, w.m[2] * z));
  r.y = fmaf(w.m[3], x, fmaf(w.m[4], y, w.m[5] * z));
  r.z = fmaf(w.m[6], x, fmaf(w.m[7], y, w.m[8] * z));
  return r;
}

// True only when no ray of the tile's rectangle can reach decay > thr against this primitive, i.e. when
// every such line stays outside the ellipsoid r^2 <= K0 = -2 ln thr.  In the primitive's whitened frame
// (rotate by R^T, divide axis k by exp(ls_k)) the ellipsoid is the sphere of radius sqrt(K0) around the
// origin and a line from x with direction e meets it iff |x cross e|^2 <= K0 |e|^2.  Both sides are
// quadratic in (alpha, beta), so q = |x cross e|^2 - K |e|^2 is minimised exactly over the rectangle
// (stationary point, four edges).  K carries a 0.2 % margin and tol bounds the rounding of this test and of
// hit_test (which works in world space, where a position error of a few ulps of |c - o| is magnified by the
// largest inverse scale); both are orders of magnitude above the error of the approximate divisions and
// square roots used here.  So a rejected pair is one hit_test rejects for every pixel of the tile, and the
// rendered result does not depend on the pre-test.  Any NaN makes the test answer false.
__device__ __forceinline__ bool tile_surely_misses(const PrimWhiten& pw, const TileFrame& f, float K0) {
  if (!(f.a0 <= f.a1)) return false;
  const float vx = pw.cx - f.ox, vy = pw.cy - f.oy, vz = pw.cz - f.oz;
  const V3 x = whiten(pw, vx, vy, vz);
  const V3 e0 = whiten(pw, f.ax, f.ay, f.az);
  const V3 e1 = whiten(pw, f.ux, f.uy, f.uz);
  const V3 e2 = whiten(pw, f.vx, f.vy, f.vz);
  const V3 w0 = {x.y * e0.z - x.z * e0.y, x.z * e0.x - x.x * e0.z, x.x * e0.y - x.y * e0.x};
  const V3 w1 = {x.y * e1.z - x.z * e1.y, x.z * e1.x - x.x * e1.z, x.x * e1.y - x.y * e1.x};
  const V3 w2 = {x.y * e2.z - x.z * e2.y, x.z * e2.x - x.x * e2.z, x.x * e2.y - x.y * e2.x};
  const float K = K0 * 1.002f;
  const float e00 = e0.x * e0.x + e0.y * e0.y + e0.z * e0.z;
  const float e11 = e1.x * e1.x + e1.y * e1.y + e1.z * e1.z;
  const float e22 = e2.x * e2.x + e2.y * e2.y + e2.z * e2.z;
  const float a11 = (w1.x * w1.x + w1.y * w1.y + w1.z * w1.z) - K * e11;
  const float a22 = (w2.x * w2.x + w2.y * w2.y + w2.z * w2.z) - K * e22;
  const float a12 = (w1.x * w2.x + w1.y * w2.y + w1.z * w2.z) - K * (e1.x * e2.x + e1.y * e2.y + e1.z * e2.z);
  const float b1 = (w0.x * w1.x + w0.y * w1.y + w0.z * w1.z) - K * (e0.x * e1.x + e0.y * e1.y + e0.z * e1.z);
  const float b2 = (w0.x * w2.x + w0.y * w2.y + w0.z * w2.z) - K * (e0.x * e2.x + e0.y * e2.y + e0.z * e2.z);
  const float c0 = (w0.x * w0.x + w0.y * w0.y + w0.z * w0.z) - K * e00;
  if (!(fabsf(a11) + fabsf(a22) + fabsf(a12) + fabsf(b1) + fabsf(b2) + fabsf(c0) < 3.0e38f)) return false;
  if (c0 <= 0.f) return false;   // the tile's central direction already reaches the ellipsoid
  // edges alpha = a0 / a1 (quadratics in beta) and beta = b0 / b1 (quadratics in alpha)
  float m = quad_min_1d(a22, fmaf(a12, f.a0, b2), fmaf(fmaf(a11, f.a0, 2.f * b1), f.a0, c0), f.b0, f.b1);
  m = fminf(m, quad_min_1d(a22, fmaf(a12, f.a1, b2), fmaf(fmaf(a11, f.a1, 2.f * b1), f.a1, c0), f.b0, f.b1));
  m = fminf(m, quad_min_1d(a11, fmaf(a12, f.b0, b1), fmaf(fmaf(a22, f.b0, 2.f * b2), f.b0, c0), f.a0, f.a1));
  m = fminf(m, quad_min_1d(a11, fmaf(a12, f.b1, b1), fmaf(fmaf(a22, f.b1, 2.f * b2), f.b1, c0), f.a0, f.a1));
  const float det = a11 * a22 - a12 * a12;
  if (a11 > 0.f && det > 0.f) {
    const float rdet = __fdividef(1.f, det);
    const float al = (a12 * b2 - a22 * b1) * rdet, be = (a12 * b1 - a11 * b2) * rdet;
    if (al >= f.a0 && al <= f.a1 && be >= f.b0 && be <= f.b1) m = fminf(m, fmaf(b1, al, fmaf(b2, be, c0)));
  }
  const float dist = sqrtf(vx * vx + vy * vy + vz * vz);
  // largest |e| over the rectangle
  const float emax = sqrtf(e00) + fmaxf(fabsf(f.a0), fabsf(f.a1)) * sqrtf(e11) +
                     fmaxf(fabsf(f.b0), fabsf(f.b1)) * sqrtf(e22);
  const float tol = (2e-5f * sqrtf(K0) * dist * pw.ismax + 1e-4f * K0) * emax * emax;
  return m > tol;
}

__device__ __forceinline__ V3 load3(const float* __restrict__ p, int64_t i) {
  V3 r = { __ldg(p + i * 3), __ldg(p + i * 3 + 1), __ldg(p + i * 3 + 2) };
  return r;
}

// pixel k (row-major inside the 8x8 tile) of a tile: image index and whether it lies inside the image
struct TilePix {
  int pix; bool valid;
};

__device__ __forceinline__ TilePix tile_pixel(int tile, int k, int ntx, int W, int H) {
  const int tx = tile % ntx, ty = tile / ntx;
  const int x = tx * 8 + (k & 7), y = ty * 8 + (k >> 3);
  TilePix r;
  r.valid = (x < W) && (y < H);
  r.pix = r.valid ? y * W + x : 0;
  return r;
}

// Output activations (np_tile_kernels.cu:75-83); values, not decisions, so hardware exp is fine.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float softplus_fast(float x) {
  if (x > 20.f) return x;
  if (x < -20.f) return __expf(x);
  // log(1 + e) on the hardware logarithm: within 1e-7 absolute of log1p over this range, far below what the
  // compositing weights resolve
  return __logf(1.0f + __expf(x));
}

// position of the (k+1)-th set bit of m (k >= 0 and fewer than popc(m)): five halvings by population count, the
// same number of steps for every lane of a warp (the library's __fns walks the set bits one by one)
__device__ __forceinline__ int nth_set_bit(uint32_t m, int k) {
  int pos = 0, c;
  c = __popc(m & 0xffffu); if (k >= c) { k -= c; pos += 16; m >>= 16; }
  c = __popc(m & 0xffu);   if (k >= c) { k -= c; pos += 8;  m >>= 8; }
  c = __popc(m & 0xfu);    if (k >= c) { k -= c; pos += 4;  m >>= 4; }
  c = __popc(m & 0x3u);    if (k >= c) { k -= c; pos += 2;  m >>= 2; }
  c = (int)(m & 1u);       if (k >= c) { pos += 1; }
  return pos;
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
