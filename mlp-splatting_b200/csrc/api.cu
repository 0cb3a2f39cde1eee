// C ABI entry points: argument checks, scratch carving and stage sequencing.
#include <cmath>
#include <cstring>
#include <vector>
#include "frame.cuh"

namespace mlpsp {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_check(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return MLPSP_OK;
  set_error("CUDA error in %s: %s", what, cudaGetErrorString(e));
  return MLPSP_E_CUDA;
}

// ---- launch accounting and optional device timing per kernel class ----
static long long g_launches[kNumKernelClasses] = {0};
static bool g_timing = false;
struct TimedSpan { cudaEvent_t a, b; int cls; };
static std::vector<TimedSpan> g_spans;
static std::vector<cudaEvent_t> g_pool;

static cudaEvent_t take_event() {
  if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

LaunchScope::LaunchScope(KernelClass k, int launches, cudaStream_t s) : slot(-1), st(s) {
  g_launches[k] += launches;
  if (g_timing) {
    TimedSpan sp{take_event(), take_event(), (int)k};
    cudaEventRecord(sp.a, st);
    g_spans.push_back(sp);
    slot = (int)g_spans.size() - 1;
  }
}
LaunchScope::~LaunchScope() {
  if (slot >= 0) cudaEventRecord(g_spans[slot].b, st);
}

// validate_tile_candidate_capacity_kernel (np_tile_kernels.cu:4485-4520)
__global__ void k_validate_lists(const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ prims, int T,
                                 int64_t M, int capacity, int n, int32_t* __restrict__ status) {
  const int64_t stride = (int64_t)blockDim.x * gridDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < T; t += stride) {
    const int s = tile_offsets[t], e = tile_offsets[t + 1];
    if (s < 0 || e < s || e > M || (t == 0 && s != 0) || (t == T - 1 && e != M)) {
      atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_BAD_OFFSETS);
      continue;
    }
    const int c = e - s;
    atomicMax(status + MLPSP_ST_MAX_TILE_LEN, c);
    if (capacity > 0 && c > capacity) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TILE_CAPACITY);
  }
  bool bad = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M; i += stride) {
    const int p = prims[i];
    bad |= p < 0 || p >= n;
  }
  if (bad) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_BAD_IDS);
}

// coarse_ok: the stage also takes 16x16 tiles (culling and per-tile ordering; the wave kernels are 8x8 only)
static int check_frame_common(const mlpsp_scene* sc, const mlpsp_frame* fr, const char* who, bool coarse_ok = false) {
  MLPSP_REQUIRE(sc && fr, MLPSP_E_ARG, "%s: null scene or frame", who);
  MLPSP_REQUIRE(fr->width > 0 && fr->height > 0, MLPSP_E_ARG, "%s: image and tile dimensions must be positive", who);
  MLPSP_REQUIRE(fr->tile == 8 || (coarse_ok && fr->tile == 16), MLPSP_E_ARG,
                coarse_ok ? "%s: tiles must be 8x8 or 16x16" : "%s: only 8x8 tiles are supported", who);
  MLPSP_REQUIRE((int64_t)fr->width * fr->height <= 2147483647LL, MLPSP_E_LIMIT,
                "%s: image dimensions exceed int32 pixel indexing", who);
  MLPSP_REQUIRE(fr->threshold > 0.f && fr->threshold < 1.f, MLPSP_E_ARG, "%s: threshold must be in (0,1)", who);
  MLPSP_REQUIRE(fr->hit_arith == 0 || fr->hit_arith == 1, MLPSP_E_ARG, "%s: hit_arith must be 0 or 1", who);
  MLPSP_REQUIRE(sc->n >= 0 && (sc->n == 0 || sc->geom), MLPSP_E_ARG, "%s: scene geometry missing", who);
  MLPSP_REQUIRE(fr->status, MLPSP_E_ARG, "%s: status block missing", who);
  MLPSP_REQUIRE(fr->tile_offsets, MLPSP_E_ARG, "%s: tile_offsets missing", who);
  MLPSP_REQUIRE(fr->max_pairs >= 0 && fr->max_pairs < (1ll << 31), MLPSP_E_LIMIT,
                "%s: candidate list is too large for int32 offsets", who);
  MLPSP_REQUIRE(fr->max_pairs == 0 || (fr->tile_prims && fr->sorted_prims), MLPSP_E_ARG, "%s: tile list buffers missing", who);
  return MLPSP_OK;
}

static int get_scratch(const mlpsp_scene* sc, const mlpsp_frame* fr, Scratch& s, const char* who) {
  MLPSP_REQUIRE(fr->max_records >= 0 && fr->max_records < (1ll << 31), MLPSP_E_LIMIT,
                "%s: max_records must be below 2^31", who);
  const Scratch q = carve_scratch(nullptr, sc->n, fr->width, fr->height, fr->tile, fr->max_pairs, fr->max_records);
  MLPSP_REQUIRE(fr->scratch && fr->scratch_bytes >= q.bytes, MLPSP_E_SCRATCH, "%s: scratch needs %lld bytes, got %lld",
                who, (long long)q.bytes, (long long)fr->scratch_bytes);
  MLPSP_REQUIRE(((uintptr_t)fr->scratch & 255u) == 0, MLPSP_E_ARG, "%s: scratch must be 256-byte aligned", who);
  s = carve_scratch(fr->scratch, sc->n, fr->width, fr->height, fr->tile, fr->max_pairs, fr->max_records);
  return MLPSP_OK;
}

static int render_sorted_checked(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st,
                                 bool lists_refined = false) {
  MLPSP_REQUIRE(fr->rays_o && fr->rays_d && fr->rgb && fr->alpha, MLPSP_E_ARG, "render: rays or outputs missing");
  MLPSP_REQUIRE(fr->precision == MLPSP_PRECISION_F32 || fr->precision == MLPSP_PRECISION_F16 ||
                    fr->precision == MLPSP_PRECISION_BF16, MLPSP_E_ARG,
                "render: unknown precision %d", fr->precision);
  MLPSP_REQUIRE(fr->num_waves >= 0 && fr->num_waves <= MLPSP_MAX_WAVES, MLPSP_E_ARG, "render: bad num_waves");
  return launch_render_sorted(sc, fr, s, st, lists_refined);
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" const char* mlpsp_last_error(void) { return g_err; }
extern "C" int mlpsp_abi_version(void) { return MLPSP_ABI_VERSION; }
extern "C" int mlpsp_struct_sizes(int32_t* scene_bytes, int32_t* frame_bytes) {
  if (scene_bytes) *scene_bytes = (int32_t)sizeof(mlpsp_scene);
  if (frame_bytes) *frame_bytes = (int32_t)sizeof(mlpsp_frame);
  return MLPSP_OK;
}

extern "C" int mlpsp_kernel_launches(int64_t* per_class, int32_t num_classes) {
  long long total = 0;
  for (int i = 0; i < kNumKernelClasses; ++i) {
    total += g_launches[i];
    if (per_class && i < num_classes) per_class[i] = g_launches[i];
  }
  return (int)(total > 2147483647LL ? 2147483647LL : total);
}

extern "C" int mlpsp_timing_enable(int32_t on) {
  g_timing = on != 0;
  return MLPSP_OK;
}

extern "C" int mlpsp_timing_collect(float* ms_per_class, int32_t num_classes) {
  MLPSP_REQUIRE(ms_per_class && num_classes >= kNumKernelClasses, MLPSP_E_ARG,
                "mlpsp_timing_collect: need room for %d classes", (int)kNumKernelClasses);
  for (int i = 0; i < num_classes; ++i) ms_per_class[i] = 0.f;
  for (auto& sp : g_spans) {
    MLPSP_CUDA_OK(cudaEventSynchronize(sp.b));
    float ms = 0.f;
    MLPSP_CUDA_OK(cudaEventElapsedTime(&ms, sp.a, sp.b));
    ms_per_class[sp.cls] += ms;
    g_pool.push_back(sp.a);
    g_pool.push_back(sp.b);
  }
  g_spans.clear();
  return MLPSP_OK;
}

extern "C" int mlpsp_status_reset(int32_t* status, void* stream) {
  MLPSP_REQUIRE(status, MLPSP_E_ARG, "mlpsp_status_reset: null pointer");
  return cuda_check(cudaMemsetAsync(status, 0, 4 * MLPSP_STATUS_WORDS, (cudaStream_t)stream), "status_reset");
}

extern "C" int64_t mlpsp_frame_scratch_bytes(int32_t n, int32_t width, int32_t height, int32_t tile,
                                             int64_t max_pairs, int64_t max_records) {
  if (n < 0 || width <= 0 || height <= 0 || tile <= 0 || max_pairs < 0 || max_records < 0) return -1;
  return carve_scratch(nullptr, n, width, height, tile, max_pairs, max_records).bytes;
}

extern "C" int mlpsp_validate_tile_lists(const int32_t* tile_offsets, const int32_t* tile_prims, int32_t num_tiles_,
                                         int64_t pairs, int32_t tile_capacity, int32_t n, int32_t* status,
                                         void* stream) {
  MLPSP_REQUIRE(tile_offsets && status && num_tiles_ > 0, MLPSP_E_ARG, "validate: tile_offsets/status missing");
  MLPSP_REQUIRE(pairs >= 0 && pairs <= 2147483647LL, MLPSP_E_LIMIT, "validate: candidate list is too large for int32 offsets");
  MLPSP_REQUIRE(pairs == 0 || tile_prims, MLPSP_E_ARG, "validate: candidate list missing");
  MLPSP_REQUIRE(n >= 0, MLPSP_E_LIMIT, "validate: primitive count is outside the supported int32 range");
  const int64_t work = std::max<int64_t>(num_tiles_, pairs);
  const int blocks = (int)std::min<int64_t>(4096, (work + 255) / 256);
  LaunchScope scope(kKMisc, 1, (cudaStream_t)stream);
  k_validate_lists<<<blocks, 256, 0, (cudaStream_t)stream>>>(tile_offsets, tile_prims, num_tiles_, pairs,
                                                            tile_capacity, n, status);
  return cuda_check(cudaGetLastError(), "validate");
}

extern "C" int mlpsp_bin_tiles(const mlpsp_scene* sc, const mlpsp_frame* fr, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_bin_tiles", /*coarse_ok=*/true);
  if (rc) return rc;
  MLPSP_REQUIRE(fr->view && fr->proj, MLPSP_E_ARG, "mlpsp_bin_tiles: view/proj matrices missing");
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_bin_tiles");
  if (rc) return rc;
  return launch_bin(sc, fr, s, (cudaStream_t)stream);
}

extern "C" int mlpsp_bin_tiles_mosaic(const mlpsp_scene* sc, const mlpsp_frame* fr, const int32_t* tile_view_ids,
                                      const float* view_matrices, int32_t num_views, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_bin_tiles_mosaic");
  if (rc) return rc;
  MLPSP_REQUIRE(fr->proj && view_matrices && tile_view_ids, MLPSP_E_ARG, "mlpsp_bin_tiles_mosaic: matrices or tile views missing");
  MLPSP_REQUIRE(num_views > 0, MLPSP_E_ARG, "view_matrices must contain at least one view");
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_bin_tiles_mosaic");
  if (rc) return rc;
  return launch_bin_mosaic(sc, fr, s, tile_view_ids, view_matrices, num_views, (cudaStream_t)stream);
}

extern "C" int mlpsp_bin_tiles_raycone(const mlpsp_scene* sc, const mlpsp_frame* fr, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_bin_tiles_raycone");
  if (rc) return rc;
  MLPSP_REQUIRE(fr->rays_o && fr->rays_d, MLPSP_E_ARG, "mlpsp_bin_tiles_raycone: rays missing");
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_bin_tiles_raycone");
  if (rc) return rc;
  return launch_bin_raycone(sc, fr, s, (cudaStream_t)stream);
}

extern "C" int mlpsp_sort_tiles(const mlpsp_scene* sc, const mlpsp_frame* fr, float* keys_out, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_sort_tiles", /*coarse_ok=*/true);
  if (rc) return rc;
  MLPSP_REQUIRE(fr->rays_o && fr->rays_d, MLPSP_E_ARG, "mlpsp_sort_tiles: rays missing");
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_sort_tiles");
  if (rc) return rc;
  // the active-tile list of the wave loop is free while the lists are being sorted
  return launch_sort(sc, fr, keys_out, (cudaStream_t)stream, false, s.active[1], s.counters + kCtrScratch + 2);
}

extern "C" int mlpsp_hit_masks(const mlpsp_scene* sc, const mlpsp_frame* fr, uint64_t* mask_geo, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_hit_masks");
  if (rc) return rc;
  MLPSP_REQUIRE(fr->rays_o && fr->rays_d && mask_geo, MLPSP_E_ARG, "mlpsp_hit_masks: rays or output missing");
  return launch_hit_masks(sc, fr, mask_geo, (cudaStream_t)stream);
}

extern "C" int mlpsp_render_sorted(const mlpsp_scene* sc, const mlpsp_frame* fr, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_render_sorted");
  if (rc) return rc;
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_render_sorted");
  if (rc) return rc;
  return render_sorted_checked(sc, fr, s, (cudaStream_t)stream);
}

extern "C" int mlpsp_render_frame(const mlpsp_scene* sc, const mlpsp_frame* fr, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_render_frame");
  if (rc) return rc;
  MLPSP_REQUIRE(fr->view && fr->proj, MLPSP_E_ARG, "mlpsp_render_frame: view/proj matrices missing");
  MLPSP_REQUIRE(fr->rays_o && fr->rays_d, MLPSP_E_ARG, "mlpsp_render_frame: rays missing");
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_render_frame");
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // consumed-record masks are indexed by position in the full sorted list, so the pre-test stays off for them
  const bool pretest = fr->tile_pretest == 0 && fr->mask_used == nullptr && fr->tile == 8;
  rc = launch_bin(sc, fr, s, st, /*order_lists=*/false, pretest);
  if (rc) return rc;
  rc = launch_sort(sc, fr, nullptr, st, /*unordered_input=*/true, s.active[1], s.counters + kCtrScratch + 2,
                   pretest ? s.tile_len : nullptr);
  if (rc) return rc;
  return render_sorted_checked(sc, fr, s, st, pretest);
}

extern "C" int mlpsp_render_frames(const mlpsp_scene* sc, const mlpsp_frame* frames, int32_t num_frames, void* stream) {
  MLPSP_REQUIRE(sc && frames && num_frames >= 1 && num_frames <= MLPSP_MAX_BATCH, MLPSP_E_ARG,
                "mlpsp_render_frames: need 1..%d frames", MLPSP_MAX_BATCH);
  std::vector<Scratch> ss((size_t)num_frames);
  const mlpsp_frame* f0 = frames;
  for (int v = 0; v < num_frames; ++v) {
    const mlpsp_frame* fr = frames + v;
    int rc = check_frame_common(sc, fr, "mlpsp_render_frames");
    if (rc) return rc;
    MLPSP_REQUIRE(fr->view && fr->proj && fr->rays_o && fr->rays_d && fr->rgb && fr->alpha, MLPSP_E_ARG,
                  "mlpsp_render_frames: frame %d lacks matrices, rays or outputs", v);
    MLPSP_REQUIRE(fr->width == f0->width && fr->height == f0->height && fr->threshold == f0->threshold &&
                      fr->precision == f0->precision && fr->tile_capacity == f0->tile_capacity &&
                      fr->hit_arith == f0->hit_arith && fr->status == f0->status, MLPSP_E_ARG,
                  "mlpsp_render_frames: frame %d differs from frame 0 in shape, threshold, precision, capacity, "
                  "arithmetic or status block", v);
    MLPSP_REQUIRE(!fr->depth_t && !fr->feat && !fr->mask_used && !fr->keep_records && !fr->stat_sum_w &&
                      fr->sort_key == 0 && fr->tile_row_begin == 0 && fr->tile_row_end == 0, MLPSP_E_ARG,
                  "mlpsp_render_frames renders rgb and alpha of whole frames in tile-centre order only (frame %d)", v);
    rc = get_scratch(sc, fr, ss[(size_t)v], "mlpsp_render_frames");
    if (rc) return rc;
  }
  MLPSP_REQUIRE(f0->precision == MLPSP_PRECISION_F32 || f0->precision == MLPSP_PRECISION_F16 ||
                    f0->precision == MLPSP_PRECISION_BF16, MLPSP_E_ARG, "render: unknown precision %d", f0->precision);
  MLPSP_REQUIRE(f0->num_waves >= 0 && f0->num_waves <= MLPSP_MAX_WAVES, MLPSP_E_ARG, "render: bad num_waves");
  cudaStream_t st = (cudaStream_t)stream;
  const bool pretest = f0->tile_pretest == 0;
  for (int v = 0; v < num_frames; ++v) {
    const mlpsp_frame* fr = frames + v;
    const Scratch& s = ss[(size_t)v];
    int rc = launch_bin(sc, fr, s, st, /*order_lists=*/false, pretest);
    if (rc) return rc;
    rc = launch_sort(sc, fr, nullptr, st, /*unordered_input=*/true, s.active[1], s.counters + kCtrScratch + 2,
                     pretest ? s.tile_len : nullptr);
    if (rc) return rc;
  }
  return launch_render_batch(sc, frames, ss.data(), num_frames, st, pretest);
}

extern "C" int mlpsp_export_records(const mlpsp_scene* sc, const mlpsp_frame* fr, int64_t* offsets, int32_t* ids,
                                    float* x6, float* raw, int32_t* relu_masks, float* gates, int64_t max_out,
                                    int32_t max_hits, int64_t* total_host, int32_t* worst_host, void* stream) {
  int rc = check_frame_common(sc, fr, "mlpsp_export_records");
  if (rc) return rc;
  MLPSP_REQUIRE(fr->keep_records == 1, MLPSP_E_ARG, "mlpsp_export_records: the frame was not rendered with keep_records = 1");
  MLPSP_REQUIRE(offsets && fr->rays_o && fr->rays_d, MLPSP_E_ARG, "mlpsp_export_records: offsets or rays missing");
  Scratch s;
  rc = get_scratch(sc, fr, s, "mlpsp_export_records");
  if (rc) return rc;
  return launch_export_records(sc, fr, s, offsets, ids, x6, raw, relu_masks, gates, max_out, max_hits, total_host,
                               worst_host, (cudaStream_t)stream);
}

// ------------------------------------------------------------ grouped evaluator on records ----
namespace mlpsp {

__global__ void k_grouped_counts(const int64_t* __restrict__ offsets, int n, int32_t* __restrict__ cnt) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) cnt[i] = (int32_t)(offsets[i + 1] - offsets[i]);
}

__global__ void k_grouped_records(const float* __restrict__ x6, int64_t R, RecIn* __restrict__ rec) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= R) return;
  RecIn r;
  r.rdx = x6[i * 6]; r.rdy = x6[i * 6 + 1]; r.rdz = x6[i * 6 + 2];
  r.dx = x6[i * 6 + 3]; r.dy = x6[i * 6 + 4]; r.dz = x6[i * 6 + 5];
  r.decay = 1.f; r.slot = (uint32_t)i;
  rec[i] = r;
}

static Scratch grouped_layout(void* base, int64_t R, int n) {
  Scratch s;
  memset(&s, 0, sizeof(s));
  char* p = (char*)base;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { char* r = p ? p + off : nullptr; off += align_up(bytes, 256); return r; };
  s.prim_cnt = (int32_t*)take(4 * 2 * ((int64_t)n + 4));
  s.prim_cursor = (int32_t*)take(4 * ((int64_t)n + 1));
  s.prim_off = (int32_t*)take(4 * ((int64_t)n + 2));
  s.scan_blk = (int32_t*)take(4 * 3 * ((int64_t)n / kPrimScanItems + 4));
  s.max_work = (int64_t)n + R / kRowsPerItem + 2;
  s.work = (int4*)take(16 * s.max_work);
  s.max_work_small = 2 * (int64_t)n + 2;
  s.work_small = (int4*)take(16 * s.max_work_small);
  s.rec_in = (RecIn*)take(32 * std::max<int64_t>(R, 1));
  s.counters = (int32_t*)take(4 * kNumCounters);
  s.bytes = off;
  return s;
}

}  // namespace mlpsp

extern "C" int64_t mlpsp_mlp_grouped_scratch_bytes(int64_t num_records, int32_t n) {
  if (num_records < 0 || n < 0) return -1;
  return grouped_layout(nullptr, num_records, n).bytes;
}

extern "C" int mlpsp_mlp_grouped(const mlpsp_scene* sc, int32_t precision, const int64_t* offsets, const float* x6,
                                 int64_t num_records, float* out4, void* scratch, int64_t scratch_bytes,
                                 int32_t* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  MLPSP_REQUIRE(sc && offsets && status && num_records >= 0, MLPSP_E_ARG, "mlpsp_mlp_grouped: bad arguments");
  MLPSP_REQUIRE(num_records < (1ll << 31), MLPSP_E_LIMIT, "mlpsp_mlp_grouped: more than 2^31-1 records");
  MLPSP_REQUIRE(num_records == 0 || (x6 && out4), MLPSP_E_ARG, "mlpsp_mlp_grouped: null record arrays");
  const int n = sc->n;
  const Scratch q = grouped_layout(nullptr, num_records, n);
  MLPSP_REQUIRE(scratch && scratch_bytes >= q.bytes, MLPSP_E_SCRATCH, "mlpsp_mlp_grouped: scratch needs %lld bytes",
                (long long)q.bytes);
  if (n == 0 || num_records == 0) return MLPSP_OK;
  Scratch s = grouped_layout(scratch, num_records, n);
  MLPSP_CUDA_OK(cudaMemsetAsync(s.counters, 0, 4 * kNumCounters, st));
  { LaunchScope scope(kKMisc, 2, st);
  k_grouped_counts<<<(n + 255) / 256, 256, 0, st>>>(offsets, n, s.prim_cnt);
  k_grouped_records<<<(unsigned)((num_records + 255) / 256), 256, 0, st>>>(x6, num_records, s.rec_in); }
  const bool tc = precision == MLPSP_PRECISION_F16 || precision == MLPSP_PRECISION_BF16;
  const bool split_small = tc && num_records < 64 * (int64_t)n;     // fewer than 64 records per primitive on average
  int rc = launch_prim_scan(s, n, 0, status, st, split_small);
  if (rc) return rc;
  if (tc)
    return launch_mlp_f16(sc, s.rec_in, s.prim_off, s.work, s.counters, (float4*)out4, nullptr, kOutSigmaRaw, status, st,
                          precision == MLPSP_PRECISION_BF16, 0, split_small ? s.work_small : nullptr);
  MLPSP_REQUIRE(precision == MLPSP_PRECISION_F32, MLPSP_E_ARG, "mlpsp_mlp_grouped: unknown precision %d", precision);
  return launch_mlp_f32(sc, s.rec_in, s.prim_off, s.work, s.counters, (float4*)out4, nullptr, kOutSigmaRaw, status, st);
}
