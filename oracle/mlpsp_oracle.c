/*
 * CPU oracle for the MLP Splatting tile-centre render path.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls this file; only the tests, the smoke
 * check and the benchmark's CPU-baseline leg do.
 *
 * It restates, in plain C and tile-major order, what the reference renderer computes:
 *   binning            scannet/cumodel.py:994-1070
 *   tile-centre key    scannet/cuda/np_tile_kernels.cu:483-518 (rotation: 416-435)
 *   stable tile sort   np_tile_kernels.cu:1914-1990 (ascending, ties keep list order, pad 1e30)
 *   hit test           np_tile_kernels.cu:659-711
 *   PE + MLP           np_tile_kernels.cu:312-380 (scalar FP32), scannet/cuda/rgb_wmma.cuh:144-199
 *                      (fp16 operands, FP32 accumulate from zero, FP32 bias afterwards)
 *   compositing        np_tile_kernels.cu:2025-2136 (trans >= 1e-3 gate, tile-wide early exit)
 *   expected depth     np_tile_kernels.cu:5712-5714
 *   feature gates      np_tile_kernels.cu:97-124, mix 6036-6075
 *   record schema      np_tile_kernels.cu:3138-3154, scannet/cuda/training_wmma.cuh:223-256
 *
 * Arithmetic contract.  Every float operation that feeds an INTEGER decision (tile overlap,
 * sort order, hit/no-hit) is an explicitly ordered IEEE-754 binary32 operation (+,-,*,/,fmaf)
 * plus det_exp() below, which is itself built only from such operations.  The CUDA kernels
 * issue the same operations in the same order, so those decisions agree bit for bit between
 * CPU and GPU.  This replaces the reference's __expf (hardware ex2.approx), whose bits no CPU
 * can reproduce; the two differ by a few ulp.  Everything downstream of the MLP (sin/cos,
 * sigmoid, softplus, blending) is ordinary float math compared within a tolerance.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/build.py).
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_SENTINEL 1e30f
#define ORC_TERM 1e-3f
#define ORC_MAXH 64
#define ORC_MAXF 16

/* ---------------------------------------------------------------- deterministic exp ---- */
/* Cody-Waite reduction by ln2 (hi/lo), degree-5 polynomial (Cephes expf coefficients),
 * scaling by an exponent built from integer bits.  Inputs below -87 give 0, above 88 +inf. */
static inline float det_exp(float x) {
  if (!(x >= -87.0f)) return (x != x) ? x : 0.0f;
  if (x > 88.0f) return INFINITY;
  const float kf = rintf(x * 1.44269504088896341f);
  float r = fmaf(kf, -0.693359375f, x);
  r = fmaf(kf, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float r2 = r * r;
  float y = fmaf(p, r2, r);
  y = y + 1.0f;
  const int k = (int)kf;
  union { uint32_t u; float f; } s;
  s.u = (uint32_t)(k + 127) << 23;
  return y * s.f;
}
float orc_det_exp(float x) { return det_exp(x); }

/* round-to-nearest-even float -> binary16 -> float (what __float2half_rn then __half2float do) */
static inline float f16_round(float x) {
  union { float f; uint32_t u; } v = { x };
  const uint32_t sign = v.u & 0x80000000u;
  uint32_t a = v.u & 0x7fffffffu;
  if (a >= 0x7f800000u) return x;                       /* inf / nan */
  if (a >= 0x477ff000u) {                               /* >= 65520 rounds to inf */
    v.u = sign | 0x7f800000u; return v.f;
  }
  if (a < 0x38800000u) {                                /* subnormal half: quantum 2^-24 */
    union { float f; uint32_t u; } t; t.u = a;
    const float q = t.f * 16777216.0f;                  /* exact scaling */
    const float rq = rintf(q);
    t.f = rq * (1.0f / 16777216.0f);
    t.u |= sign; return t.f;
  }
  const uint32_t rem = a & 0x1fffu;
  a &= ~0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (a & 0x2000u))) a += 0x2000u;
  v.u = sign | a; return v.f;
}
float orc_f16_round(float x) { return f16_round(x); }

/* round-to-nearest-even float -> bfloat16 -> float (the top 16 bits of the binary32 pattern) */
static inline float bf16_round(float x) {
  union { float f; uint32_t u; } v = { x };
  if ((v.u & 0x7fffffffu) >= 0x7f800000u) return x;     /* inf / nan */
  const uint32_t rem = v.u & 0xffffu;
  v.u &= 0xffff0000u;
  if (rem > 0x8000u || (rem == 0x8000u && (v.u & 0x10000u))) v.u += 0x10000u;   /* may carry into inf: correct */
  return v.f;
}
float orc_bf16_round(float x) { return bf16_round(x); }
/* operand rounding of the tensor-core contract: precision 1 = binary16, 2 = bfloat16 (rgb_wmma.cuh:23-73) */
static inline float lp_round(float x, int precision) { return precision == 2 ? bf16_round(x) : f16_round(x); }

/* ------------------------------------------------------------------------ geometry ---- */
typedef struct { float x, y, z; } v3;

/* rotate v by the conjugate of unit quaternion (w,x,y,z): R^T v  (np_tile_kernels.cu:416-435).
 * cross components are fma(a,b,-(c*d)); the sums are fma(w,t,v) + cross. */
static inline v3 rot_conj(float qw, float qx, float qy, float qz, v3 v) {
  const float ux = -qx, uy = -qy, uz = -qz;
  const float tx = 2.f * fmaf(uy, v.z, -(uz * v.y));
  const float ty = 2.f * fmaf(uz, v.x, -(ux * v.z));
  const float tz = 2.f * fmaf(ux, v.y, -(uy * v.x));
  v3 r;
  r.x = fmaf(qw, tx, v.x) + fmaf(uy, tz, -(uz * ty));
  r.y = fmaf(qw, ty, v.y) + fmaf(uz, tx, -(ux * tz));
  r.z = fmaf(qw, tz, v.z) + fmaf(ux, ty, -(uy * tx));
  return r;
}

/* packed primitive geometry: 16 floats
 * [0..2] centre, [3] qw, [4..6] qx qy qz, [7] max_k exp(ls_k), [8..10] m_k = exp(-2 ls_k),
 * [11] 0, [12..14] log-scales, [15] 0 */
void orc_pack_geometry(const float* pos, const float* ls, const float* quat, int n, float* geom) {
  for (int i = 0; i < n; ++i) {
    float* g = geom + (size_t)i * 16;
    g[0] = pos[i*3]; g[1] = pos[i*3+1]; g[2] = pos[i*3+2];
    g[3] = quat[i*4]; g[4] = quat[i*4+1]; g[5] = quat[i*4+2]; g[6] = quat[i*4+3];
    const float sx = det_exp(ls[i*3]), sy = det_exp(ls[i*3+1]), sz = det_exp(ls[i*3+2]);
    g[7] = fmaxf(fmaxf(sx, sy), sz);
    g[8] = det_exp(-2.f * ls[i*3]); g[9] = det_exp(-2.f * ls[i*3+1]); g[10] = det_exp(-2.f * ls[i*3+2]);
    g[11] = 0.f; g[12] = ls[i*3]; g[13] = ls[i*3+1]; g[14] = ls[i*3+2]; g[15] = 0.f;
  }
}

/* x / max(|x|, 1e-12) per row, the F.normalize contract (cumodel.py:1088, 1114);
 * norm = sqrt(fma(z,z,fma(y,y,x*x))) (dim 3) */
void orc_normalize_rows(const float* in, float* out, int64_t rows, int dim) {
  for (int64_t i = 0; i < rows; ++i) {
    const float* a = in + i * dim; float* o = out + i * dim;
    float s = a[0] * a[0];
    for (int k = 1; k < dim; ++k) s = fmaf(a[k], a[k], s);
    const float nrm = fmaxf(sqrtf(s), 1e-12f);
    for (int k = 0; k < dim; ++k) o[k] = a[k] / nrm;
  }
}

static inline float key_or_hit_ab(const float* g, v3 o, v3 d, float* numer_out) {
  v3 v = { g[0] - o.x, g[1] - o.y, g[2] - o.z };
  const v3 vl = rot_conj(g[3], g[4], g[5], g[6], v);
  const v3 dl = rot_conj(g[3], g[4], g[5], g[6], d);
  const float mx = g[8], my = g[9], mz = g[10];
  const float denom = fmaf(dl.x * dl.x, mx, fmaf(dl.y * dl.y, my, (dl.z * dl.z) * mz));
  *numer_out = fmaf(dl.x * vl.x, mx, fmaf(dl.y * vl.y, my, (dl.z * vl.z) * mz));
  return denom;
}

/* tile-centre ordering key (np_tile_kernels.cu:483-518) */
static inline float tile_key(const float* g, v3 o, v3 d) {
  float numer;
  const float denom = key_or_hit_ab(g, o, d, &numer);
  if (denom <= 1e-20f) return ORC_SENTINEL;
  const float t = numer / denom;
  return (t > 0.f) ? t : ORC_SENTINEL;
}

/* Euclidean key of render_tiles_kernel_tilecenter_order_with_t (np_tile_kernels.cu:5538-5543) */
static inline float tile_key_euclid(const float* g, v3 o, v3 d) {
  const float vx = g[0] - o.x, vy = g[1] - o.y, vz = g[2] - o.z;
  const float t = fmaf(vx, d.x, fmaf(vy, d.y, vz * d.z));
  return (t > 0.f) ? t : ORC_SENTINEL;
}

typedef struct { float t, dx, dy, dz, qx, qy, qz, decay; } hit_t;

/* rotated-ellipsoid closest approach (np_tile_kernels.cu:659-711) */
static inline int hit_test(const float* g, v3 o, v3 d, float thr, hit_t* h) {
  float numer;
  const float denom = key_or_hit_ab(g, o, d, &numer);
  if (denom <= 1e-20f) return 0;
  const float t = numer / denom;
  if (!(t > 0.f)) return 0;
  const float px = fmaf(t, d.x, o.x), py = fmaf(t, d.y, o.y), pz = fmaf(t, d.z, o.z);
  v3 dd = { g[0] - px, g[1] - py, g[2] - pz };
  const v3 q = rot_conj(g[3], g[4], g[5], g[6], dd);
  float r2 = (q.x * q.x) * g[8];
  r2 = fmaf(q.y * q.y, g[9], r2);
  r2 = fmaf(q.z * q.z, g[10], r2);
  r2 = fmaxf(r2, 0.f);
  const float decay = det_exp(-0.5f * r2);
  h->t = t; h->dx = dd.x; h->dy = dd.y; h->dz = dd.z; h->qx = q.x; h->qy = q.y; h->qz = q.z;
  h->decay = decay;
  return decay > thr;
}

/* ------------------------------------------------------------------------- binning ---- */
/* Screen-space culling of cumodel.py:994-1046 for one primitive; returns 0 when culled.
 * Tile range [tx0,tx1] x [ty0,ty1] inclusive is exactly the set of tiles passing the strict
 * overlap predicate  min < (t+1)*ts  &&  max > t*ts. */
static inline float dot4(const float* row, float x, float y, float z, float w) {
  float a = row[0] * x;
  a = fmaf(row[1], y, a);
  a = fmaf(row[2], z, a);
  a = fmaf(row[3], w, a);
  return a;
}

static int tile_span(float lo, float hi, int ts, int nt, int* t0, int* t1) {
  /* smallest t with (t+1)*ts > lo ; largest t with t*ts < hi ; NaN -> empty */
  if (!(lo == lo) || !(hi == hi)) return 0;
  const float fts = (float)ts;
  int a, b;
  if (lo < 0.f) a = 0;
  else if (lo >= (float)nt * fts) return 0;
  else { a = (int)(lo / fts); while (a > 0 && (float)(a * ts) > lo) --a; while ((float)((a + 1) * ts) <= lo) ++a; }
  if (hi <= 0.f) return 0;
  else if (hi > (float)(nt - 1) * fts) b = nt - 1;
  else { b = (int)(hi / fts); while ((float)(b * ts) >= hi) --b; while (b + 1 < nt && (float)((b + 1) * ts) < hi) ++b; }
  if (a >= nt || b < 0 || a > b) return 0;
  *t0 = a; *t1 = b;
  return 1;
}

static int prim_rect(const float* g, const float* view, const float* proj, int W, int H, int ts,
                     float radius_mult, int ntx, int nty, int rect[4]) {
  const float vx = dot4(view + 0, g[0], g[1], g[2], 1.f);
  const float vy = dot4(view + 4, g[0], g[1], g[2], 1.f);
  const float vz = dot4(view + 8, g[0], g[1], g[2], 1.f);
  const float vw = dot4(view + 12, g[0], g[1], g[2], 1.f);
  const float depth = vz;
  if (!(depth > 0.001f)) return 0;
  const float fx = (proj[0] * (float)W) / 2.0f;
  const float fy = (proj[5] * (float)H) / 2.0f;
  const float focal = (fx + fy) * 0.5f;
  const float world_r = g[7] * radius_mult;
  const float pix_r = world_r / (depth + 1e-8f) * focal;
  const float cxp = dot4(proj + 0, vx, vy, vz, vw);
  const float cyp = dot4(proj + 4, vx, vy, vz, vw);
  float cw = dot4(proj + 12, vx, vy, vz, vw);
  if (cw == 0.f) cw = cw + 1e-6f;
  const float nx = cxp / cw, ny = cyp / cw;
  const float sx = (nx + 1.f) * 0.5f * (float)W;
  const float sy = (ny + 1.f) * 0.5f * (float)H;
  if (!tile_span(sx - pix_r, sx + pix_r, ts, ntx, &rect[0], &rect[1])) return 0;
  if (!tile_span(sy - pix_r, sy + pix_r, ts, nty, &rect[2], &rect[3])) return 0;
  return 1;
}

float orc_radius_multiplier(float thr) { return (float)sqrt(-2.0 * log((double)thr)); }

/* pass 1: tile_offsets[T+1] (exclusive prefix of per-tile counts); returns total pairs */
int64_t orc_bin_count(const float* geom, int n, const float* view, const float* proj, int W, int H,
                      int ts, float thr, int32_t* tile_offsets) {
  const int ntx = (W + ts - 1) / ts, nty = (H + ts - 1) / ts;
  const int T = ntx * nty;
  const float rm = orc_radius_multiplier(thr);
  int64_t* cnt = (int64_t*)calloc((size_t)T + 1, sizeof(int64_t));
  for (int p = 0; p < n; ++p) {
    int r[4];
    if (!prim_rect(geom + (size_t)p * 16, view, proj, W, H, ts, rm, ntx, nty, r)) continue;
    for (int ty = r[2]; ty <= r[3]; ++ty)
      for (int tx = r[0]; tx <= r[1]; ++tx) cnt[ty * ntx + tx]++;
  }
  int64_t acc = 0;
  for (int t = 0; t < T; ++t) { tile_offsets[t] = (int32_t)acc; acc += cnt[t]; }
  tile_offsets[T] = (int32_t)acc;
  free(cnt);
  return acc;
}

/* pass 2: ascending primitive id inside each tile (the order nonzero() yields, cumodel.py:1054) */
void orc_bin_fill(const float* geom, int n, const float* view, const float* proj, int W, int H,
                  int ts, float thr, const int32_t* tile_offsets, int32_t* tile_prims) {
  const int ntx = (W + ts - 1) / ts, nty = (H + ts - 1) / ts;
  const int T = ntx * nty;
  const float rm = orc_radius_multiplier(thr);
  int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
  memcpy(cur, tile_offsets, sizeof(int32_t) * (size_t)T);
  for (int p = 0; p < n; ++p) {
    int r[4];
    if (!prim_rect(geom + (size_t)p * 16, view, proj, W, H, ts, rm, ntx, nty, r)) continue;
    for (int ty = r[2]; ty <= r[3]; ++ty)
      for (int tx = r[0]; tx <= r[1]; ++tx) tile_prims[cur[ty * ntx + tx]++] = p;
  }
  free(cur);
}

/* mosaic culling (cumodel.py:838-949): tile t is seen from view tile_view[t]; count (prims NULL) or fill */
int64_t orc_bin_mosaic(const float* geom, int n, const float* views, int num_views, const int32_t* tile_view,
                       const float* proj, int W, int H, int ts, float thr, int32_t* tile_offsets, int32_t* tile_prims) {
  const int ntx = (W + ts - 1) / ts, nty = (H + ts - 1) / ts;
  const int T = ntx * nty;
  const float rm = orc_radius_multiplier(thr);
  int32_t* cur = (int32_t*)calloc((size_t)T + 1, sizeof(int32_t));
  if (tile_prims) memcpy(cur, tile_offsets, sizeof(int32_t) * (size_t)T);
  for (int p = 0; p < n; ++p)
    for (int v = 0; v < num_views; ++v) {
      int r[4];
      if (!prim_rect(geom + (size_t)p * 16, views + 16 * (size_t)v, proj, W, H, ts, rm, ntx, nty, r)) continue;
      for (int ty = r[2]; ty <= r[3]; ++ty)
        for (int tx = r[0]; tx <= r[1]; ++tx) {
          const int t = ty * ntx + tx;
          if (tile_view[t] != v) continue;
          if (tile_prims) tile_prims[cur[t]++] = p; else cur[t]++;
        }
    }
  int64_t acc = 0;
  if (!tile_prims) {
    for (int t = 0; t < T; ++t) { tile_offsets[t] = (int32_t)acc; acc += cur[t]; }
    tile_offsets[T] = (int32_t)acc;
  }
  free(cur);
  return acc;
}

/* ---- ray-cone culling (scannet/camera.py:102-146) ---- */
static inline void nrm3(float x, float y, float z, float* o) {
  const float s = fmaf(z, z, fmaf(y, y, x * x));
  const float n = fmaxf(sqrtf(s), 1e-12f);
  o[0] = x / n; o[1] = y / n; o[2] = z / n;
}

/* returns status bits: 256 = a tile's rays have different origins, 512 = a cone spans >= 90 degrees.
 * tile_prims NULL: count pass (fills tile_offsets, returns total via *total). */
int orc_bin_raycone(const float* geom, int n, const float* rays_o, const float* rays_d, int W, int H, float thr,
                    int32_t* tile_offsets, int32_t* tile_prims, int64_t* total) {
  const int ntx = (W + 7) / 8, nty = (H + 7) / 8, T = ntx * nty;
  const float rm = orc_radius_multiplier(thr);
  int status = 0;
  float* cone = (float*)malloc(sizeof(float) * 8 * (size_t)T);
  for (int t = 0; t < T; ++t) {
    const int tx = t % ntx, ty = t / ntx;
    float sx = 0.f, sy = 0.f, sz = 0.f, d[3];
    int64_t p0 = 0;
    for (int k = 0; k < 64; ++k) {
      int x = tx * 8 + (k & 7), y = ty * 8 + (k >> 3);
      if (x > W - 1) x = W - 1;
      if (y > H - 1) y = H - 1;
      const int64_t pix = (int64_t)y * W + x;
      if (k == 0) p0 = pix;
      for (int c = 0; c < 3; ++c) if (fabsf(rays_o[pix*3+c] - rays_o[p0*3+c]) > 1e-6f) status |= 256;
      nrm3(rays_d[pix*3], rays_d[pix*3+1], rays_d[pix*3+2], d);
      sx = sx + d[0]; sy = sy + d[1]; sz = sz + d[2];
    }
    float a[3];
    nrm3(sx / 64.f, sy / 64.f, sz / 64.f, a);
    float cmin = 2.f;
    for (int k = 0; k < 64; ++k) {
      int x = tx * 8 + (k & 7), y = ty * 8 + (k >> 3);
      if (x > W - 1) x = W - 1;
      if (y > H - 1) y = H - 1;
      const int64_t pix = (int64_t)y * W + x;
      nrm3(rays_d[pix*3], rays_d[pix*3+1], rays_d[pix*3+2], d);
      cmin = fminf(cmin, fmaf(d[2], a[2], fmaf(d[1], a[1], d[0] * a[0])));
    }
    cmin = fminf(1.f, fmaxf(-1.f, cmin));
    if (!(cmin > 0.f)) status |= 512;
    float* c = cone + (size_t)t * 8;
    c[0] = rays_o[p0*3]; c[1] = rays_o[p0*3+1]; c[2] = rays_o[p0*3+2]; c[3] = a[0]; c[4] = a[1]; c[5] = a[2];
    c[6] = cmin; c[7] = sqrtf(fmaxf(1.f - cmin * cmin, 0.f));
  }
  int64_t acc = 0;
  if (!status) {
    for (int t = 0; t < T; ++t) {
      const float* c = cone + (size_t)t * 8;
      if (!tile_prims) tile_offsets[t] = (int32_t)acc;
      int64_t w = tile_prims ? tile_offsets[t] : 0;
      for (int p = 0; p < n; ++p) {
        const float* g = geom + (size_t)p * 16;
        const float radius = (g[7] * rm) * 1.00001f + 1e-7f;
        const float dx = g[0] - c[0], dy = g[1] - c[1], dz = g[2] - c[2];
        const float dist = sqrtf(fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
        const float dc = fmaxf(dist, 1e-20f);
        const float ratio = fminf(1.f, fmaxf(0.f, radius / dc));
        const float cos_b = fmaf(dz, c[5], fmaf(dy, c[4], dx * c[3])) / dc;
        const float bound = c[6] * sqrtf(fmaxf(1.f - ratio * ratio, 0.f)) - c[7] * ratio;
        if ((dist <= radius) || (cos_b >= bound - 2e-6f)) {
          if (tile_prims) tile_prims[w++] = p;
          ++acc;
        }
      }
    }
    if (!tile_prims) tile_offsets[T] = (int32_t)acc;
  }
  free(cone);
  if (total) *total = acc;
  return status;
}

/* list validation (np_tile_kernels.cu:4485-4520): bit1 offsets, bit2 capacity, bit4 ids */
void orc_validate_lists(const int32_t* tile_offsets, const int32_t* prims, int T, int M, int capacity,
                        int n, int32_t status[2]) {
  status[0] = 0; status[1] = 0;
  for (int t = 0; t < T; ++t) {
    const int s = tile_offsets[t], e = tile_offsets[t + 1];
    if (s < 0 || e < s || e > M || (t == 0 && s != 0) || (t == T - 1 && e != M)) { status[0] |= 1; continue; }
    if (capacity > 0 && e - s > capacity) { status[0] |= 2; if (e - s > status[1]) status[1] = e - s; }
  }
  for (int i = 0; i < M; ++i) if (prims[i] < 0 || prims[i] >= n) { status[0] |= 4; break; }
}

/* ---------------------------------------------------------------------------- sort ---- */
typedef struct { float key; int32_t pos; int32_t id; } sort_item;
static int cmp_item(const void* a, const void* b) {
  const sort_item* x = (const sort_item*)a; const sort_item* y = (const sort_item*)b;
  if (x->key < y->key) return -1;
  if (x->key > y->key) return 1;
  return (x->pos > y->pos) - (x->pos < y->pos);
}

static inline v3 ld3(const float* p, int64_t i) { v3 r = { p[i*3], p[i*3+1], p[i*3+2] }; return r; }

/* per-tile stable ascending sort by the tile-centre key; keys_out may be NULL */
void orc_sort_tiles(const float* rays_o, const float* rays_d, const float* geom, int n,
                    const int32_t* tile_offsets, const int32_t* tile_prims, int W, int H, int ts,
                    int32_t* sorted_prims, float* keys_out, int key_mode) {
  const int ntx = (W + ts - 1) / ts, nty = (H + ts - 1) / ts;
  #pragma omp parallel for schedule(dynamic, 8)
  for (int tile = 0; tile < ntx * nty; ++tile) {
    const int tx = tile % ntx, ty = tile / ntx;
    const int s = tile_offsets[tile], e = tile_offsets[tile + 1];
    if (e <= s) continue;
    int cx = tx * ts + (ts >> 1); if (cx > W - 1) cx = W - 1;
    int cy = ty * ts + (ts >> 1); if (cy > H - 1) cy = H - 1;
    const int64_t pc = (int64_t)cy * W + cx;
    const v3 o = ld3(rays_o, pc), d = ld3(rays_d, pc);
    sort_item* it = (sort_item*)malloc(sizeof(sort_item) * (size_t)(e - s));
    for (int i = s; i < e; ++i) {
      const int p = tile_prims[i];
      float k = ORC_SENTINEL;
      if (p >= 0 && p < n) k = key_mode ? tile_key_euclid(geom + (size_t)p * 16, o, d) : tile_key(geom + (size_t)p * 16, o, d);
      it[i - s].key = k; it[i - s].pos = i - s; it[i - s].id = p;
    }
    qsort(it, (size_t)(e - s), sizeof(sort_item), cmp_item);
    for (int i = s; i < e; ++i) { sorted_prims[i] = it[i - s].id; if (keys_out) keys_out[i] = it[i - s].key; }
    free(it);
  }
}

/* ----------------------------------------------------------------------------- MLP ---- */
typedef struct {
  const float *W1, *b1, *W2, *b2, *W3, *b3;   /* [N,H,IN] [N,H] [N,H,H] [N,H] [N,4,H] [N,4] */
  const float *freq, *att;                    /* [F] */
  int F, H, IN;
  int precision;                              /* 0 = FP32 scalar order, 1 = fp16 operands */
} mlp_t;

typedef struct { float R, G, B, sigma_raw, sigma_logit; uint32_t m1, m2; } mlp_out;

static inline float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
static inline float softplus_f(float x) {
  if (x > 20.f) return x;
  if (x < -20.f) return expf(x);
  return log1pf(expf(x));
}

static void mlp_eval(const mlp_t* m, int p, const float v6[6], mlp_out* o) {
  const int H = m->H, IN = m->IN, F = m->F, half = IN / 2;
  const float* W1 = m->W1 + (size_t)p * H * IN; const float* b1 = m->b1 + (size_t)p * H;
  const float* W2 = m->W2 + (size_t)p * H * H;  const float* b2 = m->b2 + (size_t)p * H;
  const float* W3 = m->W3 + (size_t)p * 4 * H;  const float* b3 = m->b3 + (size_t)p * 4;
  float enc[2 * 6 * ORC_MAXF];
  for (int c = 0; c < 6; ++c)
    for (int f = 0; f < F; ++f) {
      const float ph = v6[c] * m->freq[f] * m->att[f];
      enc[c * F + f] = sinf(ph);
      enc[c * F + f + half] = cosf(ph);
    }
  float h1[ORC_MAXH], h2[ORC_MAXH], out[4];
  uint32_t m1 = 0, m2 = 0;
  if (m->precision == 0) {
    /* scalar order: start from the bias, fma over (c,f): sin weight then cos weight */
    for (int h = 0; h < H; ++h) {
      float a = b1[h];
      for (int j = 0; j < half; ++j) {
        a = fmaf(W1[h * IN + j], enc[j], a);
        a = fmaf(W1[h * IN + j + half], enc[j + half], a);
      }
      if (a > 0.f && h < 32) m1 |= 1u << h;
      h1[h] = a > 0.f ? a : 0.f;
    }
    for (int q = 0; q < H; ++q) {
      float a = 0.f;                      /* row_dot_vec then "+= bias" (np_tile_kernels.cu:350-353) */
      for (int h = 0; h < H; ++h) a = fmaf(W2[q * H + h], h1[h], a);
      a = b2[q] + a;
      if (a > 0.f && q < 32) m2 |= 1u << q;
      h2[q] = a > 0.f ? a : 0.f;
    }
    for (int c = 0; c < 4; ++c) {
      float a = b3[c];
      for (int h = 0; h < H; ++h) a = fmaf(W3[c * H + h], h2[h], a);
      out[c] = a;
    }
  } else {
    /* tensor-core contract: operands rounded to binary16 (precision 1) or bfloat16 (precision 2), FP32
     * accumulate from zero over ascending k, FP32 bias added afterwards, hidden activations re-rounded */
    const int pr = m->precision;
    float e16[2 * 6 * ORC_MAXF];
    for (int j = 0; j < IN; ++j) e16[j] = lp_round(enc[j], pr);
    for (int h = 0; h < H; ++h) {
      float a = 0.f;
      for (int j = 0; j < IN; ++j) a = fmaf(lp_round(W1[h * IN + j], pr), e16[j], a);
      a = a + b1[h];
      if (a > 0.f && h < 32) m1 |= 1u << h;
      h1[h] = lp_round(fmaxf(a, 0.f), pr);
    }
    for (int q = 0; q < H; ++q) {
      float a = 0.f;
      for (int h = 0; h < H; ++h) a = fmaf(lp_round(W2[q * H + h], pr), h1[h], a);
      a = a + b2[q];
      if (a > 0.f && q < 32) m2 |= 1u << q;
      h2[q] = lp_round(fmaxf(a, 0.f), pr);
    }
    for (int c = 0; c < 4; ++c) {
      float a = 0.f;
      for (int h = 0; h < H; ++h) a = fmaf(lp_round(W3[c * H + h], pr), h2[h], a);
      out[c] = a + b3[c];
    }
  }
  o->R = sigmoid_f(out[0]); o->G = sigmoid_f(out[1]); o->B = sigmoid_f(out[2]);
  o->sigma_raw = softplus_f(out[3]); o->sigma_logit = out[3]; o->m1 = m1; o->m2 = m2;
}

/* standalone evaluator for pinning against the reference's _encode_x6/_mlp_forward_indexed */
void orc_mlp_eval(const float* W1, const float* b1, const float* W2, const float* b2, const float* W3,
                  const float* b3, const float* freq, const float* att, int F, int H, int precision,
                  const int32_t* prim_ids, const float* x6, int64_t count, float* out_rgb_sigma) {
  mlp_t m = { W1, b1, W2, b2, W3, b3, freq, att, F, H, 12 * F, precision };
  #pragma omp parallel for
  for (int64_t i = 0; i < count; ++i) {
    mlp_out o; mlp_eval(&m, prim_ids[i], x6 + i * 6, &o);
    out_rgb_sigma[i*4] = o.R; out_rgb_sigma[i*4+1] = o.G; out_rgb_sigma[i*4+2] = o.B; out_rgb_sigma[i*4+3] = o.sigma_raw;
  }
}

/* tetrahedral soft gates (np_tile_kernels.cu:97-124) */
static void tetra_gates(const hit_t* h, const float* g, float beta, float tau, float gt[4]) {
  const float sx = det_exp(g[12]), sy = det_exp(g[13]), sz = det_exp(g[14]);
  float ux = h->qx / (beta * sx + 1e-6f), uy = h->qy / (beta * sy + 1e-6f), uz = h->qz / (beta * sz + 1e-6f);
  ux = fminf(1.f, fmaxf(-1.f, ux)); uy = fminf(1.f, fmaxf(-1.f, uy)); uz = fminf(1.f, fmaxf(-1.f, uz));
  const float l0 = tau * (ux + uy + uz), l1 = tau * (ux - uy - uz);
  const float l2 = tau * (-ux + uy - uz), l3 = tau * (-ux - uy + uz);
  const float lm = fmaxf(fmaxf(l0, l1), fmaxf(l2, l3));
  const float e0 = expf(l0 - lm), e1 = expf(l1 - lm), e2 = expf(l2 - lm), e3 = expf(l3 - lm);
  const float inv = 1.f / fmaxf(e0 + e1 + e2 + e3, 1e-8f);
  gt[0] = e0 * inv; gt[1] = e1 * inv; gt[2] = e2 * inv; gt[3] = e3 * inv;
}

/* -------------------------------------------------------------------------- render ---- */
typedef struct {
  const float *rays_o, *rays_d;               /* [P,3]; rays_d already normalised */
  const float* geom;                          /* [N,16] packed */
  int n;
  const int32_t *tile_offsets, *sorted_prims; /* depth-sorted lists */
  int W, H, ts;
  float thr;
  mlp_t mlp;
  const float* feat_attr; int feat_slots, feat_dim; float beta, tau;  /* optional */
  int tile_begin, tile_end;                   /* tile range to render (baseline sampling) */
  /* outputs (any may be NULL) */
  float *rgb, *alpha, *depth_t, *feat;        /* [P,3] [P] [P] [P,C] */
  uint64_t *mask_geo, *mask_used;             /* per pair, bit = ly*8+lx (tile size 8 only) */
  float* min_margin;                          /* [P] min |trans-1e-3|/1e-3 over termination tests */
  int32_t* rec_count;                         /* [P] consumed records per pixel */
  /* record emission (second call, with rec_offsets from rec_count) */
  const int64_t* rec_offsets;
  int32_t* rec_ids; float* rec_x6; float* rec_raw; int32_t* rec_masks; float* rec_gates;
  /* per-primitive contribution statistics of render_tiles_kernel_tilecenter_stats (np_tile_kernels.cu:2143-2500),
     accumulated into the caller's arrays; all NULL or all set */
  const float* gt_rgb;                        /* [P,3] */
  float *stat_sum_w, *stat_max_w; int32_t* stat_hits; float* stat_sum_werr; int32_t* stat_contrib;   /* [N] */
  int64_t evals;                              /* out: MLP evaluations performed */
} render_t;

void orc_render(render_t* a) {
  const int ts = a->ts, W = a->W, H = a->H;
  const int ntx = (W + ts - 1) / ts;
  const int npx = ts * ts;
  int64_t evals = 0;
  #pragma omp parallel for schedule(dynamic, 4) reduction(+:evals)
  for (int tile = a->tile_begin; tile < a->tile_end; ++tile) {
    const int tx = tile % ntx, ty = tile / ntx;
    const int s = a->tile_offsets[tile], e = a->tile_offsets[tile + 1];
    float trans[256], C[256][3], tacc[256], wacc[256], marg[256];
    int used[256], valid[256]; int64_t pixi[256];
    for (int k = 0; k < npx; ++k) {
      const int x = tx * ts + k % ts, y = ty * ts + k / ts;
      valid[k] = (x < W && y < H);
      pixi[k] = valid[k] ? (int64_t)y * W + x : 0;
      trans[k] = 1.f; C[k][0] = C[k][1] = C[k][2] = 0.f; tacc[k] = wacc[k] = 0.f; used[k] = 0; marg[k] = 1e30f;
      if (valid[k] && a->feat) memset(a->feat + pixi[k] * a->feat_dim, 0, sizeof(float) * (size_t)a->feat_dim);
    }
    int alive = 1;
    for (int i = s; i < e; ++i) {
      const int p = a->sorted_prims[i];
      uint64_t mg = 0, mu = 0;
      float t_sum_w = 0.f, t_max_w = 0.f, t_sum_werr = 0.f; int t_hits = 0, t_contrib = 0;
      if (p >= 0 && p < a->n) {
        const float* g = a->geom + (size_t)p * 16;
        for (int k = 0; k < npx; ++k) {
          if (!valid[k]) continue;
          const v3 o = ld3(a->rays_o, pixi[k]), d = ld3(a->rays_d, pixi[k]);
          hit_t h;
          const int hit = hit_test(g, o, d, a->thr, &h);
          if (hit && ts == 8) mg |= 1ull << k;
          if (!alive || !hit) continue;
          if (!(trans[k] >= ORC_TERM)) continue;
          if (ts == 8) mu |= 1ull << k;
          const float v6[6] = { d.x, d.y, d.z, h.dx, h.dy, h.dz };
          mlp_out mo; mlp_eval(&a->mlp, p, v6, &mo); ++evals;
          const float sigma = mo.sigma_raw * h.decay;
          const float al = 1.f - expf(-sigma);
          const float w = trans[k] * al;
          if (a->rec_ids && a->rec_offsets) {
            const int64_t r = a->rec_offsets[pixi[k]] + used[k];
            a->rec_ids[r] = p;
            for (int c = 0; c < 6; ++c) a->rec_x6[r*6+c] = v6[c];
            float* raw = a->rec_raw + r * 8;
            raw[0] = mo.R; raw[1] = mo.G; raw[2] = mo.B; raw[3] = mo.sigma_raw;
            raw[4] = trans[k]; raw[5] = al; raw[6] = h.decay; raw[7] = mo.sigma_logit;
            a->rec_masks[r*2] = (int32_t)mo.m1; a->rec_masks[r*2+1] = (int32_t)mo.m2;
            tetra_gates(&h, g, a->beta, a->tau, a->rec_gates + r * 4);
          }
          C[k][0] = fmaf(w, mo.R, C[k][0]); C[k][1] = fmaf(w, mo.G, C[k][1]); C[k][2] = fmaf(w, mo.B, C[k][2]);
          tacc[k] = fmaf(w, h.t, tacc[k]); wacc[k] += w;
          if (a->stat_sum_w) {
            /* np_tile_kernels.cu:2391-2410: hit when w > 1e-8, "significant" when w > 0.1; the error is the L1
               distance of the partial colour after this record to the ground truth */
            const float* gt = a->gt_rgb + pixi[k] * 3;
            const float err = fabsf(C[k][0] - gt[0]) + fabsf(C[k][1] - gt[1]) + fabsf(C[k][2] - gt[2]);
            t_sum_w += w; if (w > t_max_w) t_max_w = w;
            if (w > 1e-8f) ++t_hits;
            if (w > 1e-1f) { ++t_contrib; t_sum_werr += w * err; }
          }
          if (a->feat) {
            const int Cf = a->feat_dim, S = a->feat_slots;
            float* dst = a->feat + pixi[k] * Cf;
            const float* fa = a->feat_attr + (size_t)p * S * Cf;
            if (S <= 1) { for (int c = 0; c < Cf; ++c) dst[c] = fmaf(w, fa[c], dst[c]); }
            else {
              float gt[4]; tetra_gates(&h, g, a->beta, a->tau, gt);
              const int b = (S == 5) ? 1 : 0;
              for (int c = 0; c < Cf; ++c) {
                float mix = (S == 5) ? fa[c] : 0.f;
                mix = fmaf(gt[0], fa[(b + 0) * Cf + c], mix); mix = fmaf(gt[1], fa[(b + 1) * Cf + c], mix);
                mix = fmaf(gt[2], fa[(b + 2) * Cf + c], mix); mix = fmaf(gt[3], fa[(b + 3) * Cf + c], mix);
                dst[c] = fmaf(w, mix, dst[c]);
              }
            }
          }
          trans[k] = trans[k] * (1.f - al);
          used[k]++;
          const float mrel = fabsf(trans[k] - ORC_TERM) / ORC_TERM;
          if (mrel < marg[k]) marg[k] = mrel;
        }
      }
      if (a->mask_geo) a->mask_geo[i] = mg;
      if (a->mask_used) a->mask_used[i] = mu;
      if (a->stat_sum_w && mu) {
        #pragma omp critical(orc_stats)
        {
          a->stat_sum_w[p] += t_sum_w; if (t_max_w > a->stat_max_w[p]) a->stat_max_w[p] = t_max_w;
          a->stat_hits[p] += t_hits; a->stat_sum_werr[p] += t_sum_werr; a->stat_contrib[p] += t_contrib;
        }
      }
      if (alive) {
        int any = 0;
        for (int k = 0; k < npx; ++k) any |= (valid[k] && trans[k] >= ORC_TERM);
        if (!any) { alive = 0; if (!a->mask_geo) break; }
      }
    }
    for (int k = 0; k < npx; ++k) {
      if (!valid[k]) continue;
      const int64_t px = pixi[k];
      if (a->rgb) { a->rgb[px*3] = C[k][0]; a->rgb[px*3+1] = C[k][1]; a->rgb[px*3+2] = C[k][2]; }
      if (a->alpha) a->alpha[px] = 1.f - trans[k];
      if (a->depth_t) a->depth_t[px] = tacc[k] / ((wacc[k] > 1e-8f) ? wacc[k] : 1.f);
      if (a->min_margin) a->min_margin[px] = marg[k];
      if (a->rec_count) a->rec_count[px] = used[k];
    }
  }
  a->evals = evals;
}

int orc_sizeof_render(void) { return (int)sizeof(render_t); }
int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
/* Thread count of the parallel loops from here on (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ---------------------------------------------------------------------------------------------
 * Feature decoder and text query: the step that follows the feature map.
 * ------------------------------------------------------------------------------------------- */

/* Conv 1x1 -> ReLU -> conv 3x3 (zero padding 1) -> ReLU -> conv 1x1 (scannet/feature_decoder.py:5-19), on a
 * pixel-major map x[H][W][Cin] as the renderer writes it (the reference permutes to NCHW first,
 * scannet/eval_lseg_table2.py:1221-1225).  Weights in torch Conv2d layout: W1 [Ch][Cin], W2 [Ch][Ch][3][3],
 * W3 [Cout][Ch].  precision 0: FP32 throughout; 1 / 2: inputs, weights and hidden activations rounded to
 * binary16 / bfloat16, FP32 accumulation from zero, FP32 bias added afterwards (the tensor-core contract of
 * scannet/cuda/rgb_wmma.cuh:75-223 applied to this network).  out[H*W][Cout]. */
void orc_decode_features(const float* x, int W, int H, int Cin, int Ch, int Cout,
                         const float* W1, const float* b1, const float* W2, const float* b2,
                         const float* W3, const float* b3, int precision, float* out) {
  const int64_t P = (int64_t)W * H;
  float* h1 = (float*)malloc(sizeof(float) * (size_t)P * Ch);
  float* h2 = (float*)malloc(sizeof(float) * (size_t)P * Ch);
  float* w1 = (float*)malloc(sizeof(float) * (size_t)Ch * Cin);
  float* w2 = (float*)malloc(sizeof(float) * (size_t)Ch * Ch * 9);
  float* w3 = (float*)malloc(sizeof(float) * (size_t)Cout * Ch);
  for (int64_t i = 0; i < (int64_t)Ch * Cin; ++i) w1[i] = precision ? lp_round(W1[i], precision) : W1[i];
  for (int64_t i = 0; i < (int64_t)Ch * Ch * 9; ++i) w2[i] = precision ? lp_round(W2[i], precision) : W2[i];
  for (int64_t i = 0; i < (int64_t)Cout * Ch; ++i) w3[i] = precision ? lp_round(W3[i], precision) : W3[i];
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < P; ++p) {
    for (int j = 0; j < Ch; ++j) {
      float acc = 0.0f;
      for (int k = 0; k < Cin; ++k) {
        const float v = precision ? lp_round(x[p * Cin + k], precision) : x[p * Cin + k];
        acc += v * w1[(int64_t)j * Cin + k];
      }
      acc += b1[j];
      acc = acc > 0.0f ? acc : 0.0f;
      h1[p * Ch + j] = precision ? lp_round(acc, precision) : acc;
    }
  }
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < P; ++p) {
    const int py = (int)(p / W), px = (int)(p % W);
    for (int j = 0; j < Ch; ++j) {
      float acc = 0.0f;
      for (int dy = -1; dy <= 1; ++dy) {
        const int y = py + dy;
        if (y < 0 || y >= H) continue;
        for (int dx = -1; dx <= 1; ++dx) {
          const int xx = px + dx;
          if (xx < 0 || xx >= W) continue;
          const float* hrow = h1 + ((int64_t)y * W + xx) * Ch;
          const float* wrow = w2 + (int64_t)j * Ch * 9 + (dy + 1) * 3 + (dx + 1);
          for (int k = 0; k < Ch; ++k) acc += hrow[k] * wrow[(int64_t)k * 9];
        }
      }
      acc += b2[j];
      acc = acc > 0.0f ? acc : 0.0f;
      h2[p * Ch + j] = precision ? lp_round(acc, precision) : acc;
    }
  }
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < P; ++p) {
    for (int j = 0; j < Cout; ++j) {
      float acc = 0.0f;
      for (int k = 0; k < Ch; ++k) acc += h2[p * Ch + k] * w3[(int64_t)j * Ch + k];
      out[p * Cout + j] = acc + b3[j];
    }
  }
  free(h1); free(h2); free(w1); free(w2); free(w3);
}

/* Text query of a feature map (scannet/eval_lseg_table2.py:622-641): rows of both sides divided by
 * max(||row||, 1e-12) (torch.nn.functional.normalize), logits = feature . text, label = index of the first
 * maximum.  margin (optional) = best logit - second best (0 with a single class). */
void orc_classify_features(const float* feat, int64_t P, int D, const float* text, int C,
                           int64_t* labels, float* margin) {
  float* tn = (float*)malloc(sizeof(float) * (size_t)C * D);
  for (int c = 0; c < C; ++c) {
    double s = 0.0;
    for (int k = 0; k < D; ++k) s += (double)text[(int64_t)c * D + k] * text[(int64_t)c * D + k];
    float nrm = (float)sqrt(s);
    if (nrm < 1e-12f) nrm = 1e-12f;
    for (int k = 0; k < D; ++k) tn[(int64_t)c * D + k] = text[(int64_t)c * D + k] / nrm;
  }
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < P; ++p) {
    const float* f = feat + p * D;
    double s = 0.0;
    for (int k = 0; k < D; ++k) s += (double)f[k] * f[k];
    float nrm = (float)sqrt(s);
    if (nrm < 1e-12f) nrm = 1e-12f;
    float best = 0.0f, second = 0.0f;
    int arg = -1;
    for (int c = 0; c < C; ++c) {
      float acc = 0.0f;
      for (int k = 0; k < D; ++k) acc += (f[k] / nrm) * tn[(int64_t)c * D + k];
      if (arg < 0) { best = acc; arg = c; second = -3.0e38f; }
      else if (acc > best) { second = best; best = acc; arg = c; }
      else if (acc > second) second = acc;
    }
    labels[p] = arg;
    if (margin) margin[p] = C > 1 ? best - second : 0.0f;
  }
  free(tn);
}

/* ---------------------------------------------------------------------------------------------
 * Per-pixel exact ordering (render_tiles_kernel_with_sort, np_tile_kernels.cu:714-926): every pixel gathers
 * its own hits from its tile's candidate list (at most 256; one more sets *overflow and the pixel blends the
 * 256 it has, as the kernel's loop does before its wrapper raises), sorts them by its own hit distance t with
 * a stable insertion sort (ties keep list order) and blends front to back until the transmittance falls
 * below 1e-3.  prims is the tile's list in any order.
 * ------------------------------------------------------------------------------------------- */
void orc_render_per_pixel(const float* rays_o, const float* rays_d, const float* geom, int n,
                          const int32_t* tile_offsets, const int32_t* prims, int W, int H, int ts, float thr,
                          const mlp_t* mlp, float* rgb, float* alpha, int32_t* hits_per_pixel, int32_t* overflow,
                          const float* feat_attr, int feat_slots, int feat_dim, float beta, float tau, float* feat) {
  const int ntx = (W + ts - 1) / ts;
  int any_overflow = 0;
  #pragma omp parallel for schedule(dynamic, 64) reduction(|:any_overflow)
  for (int64_t pix = 0; pix < (int64_t)W * H; ++pix) {
    const int x = (int)(pix % W), y = (int)(pix / W);
    const int tile = (y / ts) * ntx + x / ts;
    const v3 o = ld3(rays_o, pix), d = ld3(rays_d, pix);
    float ht[256]; int hp[256]; hit_t hh[256];
    int cnt = 0;
    for (int i = tile_offsets[tile]; i < tile_offsets[tile + 1]; ++i) {
      const int p = prims[i];
      if (p < 0 || p >= n) continue;
      hit_t h;
      if (!hit_test(geom + (size_t)p * 16, o, d, thr, &h)) continue;
      if (cnt >= 256) { any_overflow = 1; break; }
      ht[cnt] = h.t; hp[cnt] = p; hh[cnt] = h; ++cnt;
    }
    if (hits_per_pixel) hits_per_pixel[pix] = cnt;
    for (int i = 1; i < cnt; ++i) {
      const float kt = ht[i]; const int kp = hp[i]; const hit_t kh = hh[i];
      int j = i - 1;
      while (j >= 0 && ht[j] > kt) { ht[j + 1] = ht[j]; hp[j + 1] = hp[j]; hh[j + 1] = hh[j]; --j; }
      ht[j + 1] = kt; hp[j + 1] = kp; hh[j + 1] = kh;
    }
    float C0 = 0.f, C1 = 0.f, C2 = 0.f, trans = 1.f;
    for (int i = 0; i < cnt; ++i) {
      const float v6[6] = { d.x, d.y, d.z, hh[i].dx, hh[i].dy, hh[i].dz };
      mlp_out mo; mlp_eval(mlp, hp[i], v6, &mo);
      const float al = 1.f - expf(-(mo.sigma_raw * hh[i].decay));
      const float w = trans * al;
      C0 = fmaf(w, mo.R, C0); C1 = fmaf(w, mo.G, C1); C2 = fmaf(w, mo.B, C2);
      if (feat) {
        /* the gated attribute mix of the tile-centre feature kernel (np_tile_kernels.cu:97-124, 6036-6075), which
           render_tiles_kernel_with_sort_and_feat applies in the per-pixel order */
        const int Cf = feat_dim, S = feat_slots;
        float* dst = feat + pix * Cf;
        const float* fa = feat_attr + (size_t)hp[i] * S * Cf;
        if (S <= 1) { for (int c = 0; c < Cf; ++c) dst[c] = fmaf(w, fa[c], dst[c]); }
        else {
          float gt[4]; tetra_gates(&hh[i], geom + (size_t)hp[i] * 16, beta, tau, gt);
          const int b = (S == 5) ? 1 : 0;
          for (int c = 0; c < Cf; ++c) {
            float mix = (S == 5) ? fa[c] : 0.f;
            mix = fmaf(gt[0], fa[(b + 0) * Cf + c], mix); mix = fmaf(gt[1], fa[(b + 1) * Cf + c], mix);
            mix = fmaf(gt[2], fa[(b + 2) * Cf + c], mix); mix = fmaf(gt[3], fa[(b + 3) * Cf + c], mix);
            dst[c] = fmaf(w, mix, dst[c]);
          }
        }
      }
      trans *= (1.f - al);
      if (trans < ORC_TERM) break;
    }
    rgb[pix * 3] = C0; rgb[pix * 3 + 1] = C1; rgb[pix * 3 + 2] = C2;
    alpha[pix] = 1.f - trans;
  }
  if (overflow) *overflow = any_overflow;
}
