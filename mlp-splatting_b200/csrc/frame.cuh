// Scratch layout of one frame and small host helpers shared by the stage launchers.
#pragma once
#include <algorithm>
#include <cstdio>
#include <cstdarg>
#include <utility>
#include "common.cuh"

namespace mlpsp {

// Rows handled by one evaluator work item (one tensor-core M tile), and by an item of the small-group list.
constexpr int kRowsPerItem = 128;
constexpr int kRowsPerSmallItem = 32;
// counters[] slots (device int32)
enum Counter {
  kCtrRecords = 0,   // records appended by the hit pass of the current wave
  kCtrWork = 1,      // evaluator work items of the current wave
  kCtrWorkNext = 2,  // dynamic work cursor of the evaluator
  kCtrActive0 = 3,   // active tile count, list 0
  kCtrActive1 = 4,   // active tile count, list 1
  kCtrPairs = 5,     // total candidate pairs (binning)
  kCtrScratch = 6,   // three words (record export, long-tile list of the sort)
  kCtrWorkSmall = 10, // small-group work items of the current wave
  kNumCounters = 16
};

// One evaluator input record (32 bytes): encoded-input vector, decay and the compositing slot.
struct __align__(16) RecIn {
  float rdx, rdy, rdz, dx;
  float dy, dz, decay;
  uint32_t slot;
};

struct Scratch {
  int32_t* tile_cnt;     // [T+1]
  int32_t* tile_diff;    // [(nty+1)*(ntx+1)] rectangle corners of the count pass (2-D difference array)
  int32_t* tile_fill;    // [T]
  uint2* rect;           // [n]  (x0 | x1<<16, y0 | y1<<16); x0 > x1 marks "culled"
  int32_t* scan_blk;     // block sums of the multi-block scans
  float4* px_state;      // [P] (C.r, C.g, C.b, transmittance)
  float2* px_depth;      // [P] (sum w t, sum w)
  uint32_t* masks32;     // [2*max_pairs] evaluated-hit mask halves per pair
  uint32_t* pair_base;   // [max_pairs] first compositing slot of the pair
  int32_t* prim_cnt;     // [2][n] records per primitive in the current wave (even waves use the first half, odd the second)
  int32_t* prim_cursor;  // [n]
  int32_t* prim_off;     // [n+1]
  int4* work;            // [max_work] (primitive, first record, rows, 0)
  int4* work_small;      // [max_work_small] the same for items of at most kRowsPerSmallItem rows
  RecIn* rec_in;         // [max_records] primitive-major, reused by every wave
  float4* rec_out;       // [max_records] (R,G,B,alpha) at compositing slots (slots are unique per frame)
  float* rec_t;          // [max_records] t* at compositing slots
  float4* rec_gate;      // [max_records] feature gates at compositing slots
  float* rec_w;          // [max_records] compositing weight trans*alpha of consumed records
  float* rec_tr;         // [max_records] transmittance before the record (record export)
  float4* rec_ext;       // [max_records] (sigma_raw, sigma_logit, relu mask 1, relu mask 2) (record export)
  int32_t* px_cnt;       // [P+2] per-pixel record counts (record export)
  int32_t* px_off;       // [P+2] their exclusive prefix
  uint32_t* used32;      // [2*max_pairs] consumed-record mask halves per pair (when the caller gives none)
  int32_t* active[2];    // [T] each
  TileFrame* tile_frame; // [T] ray frame of every tile (tile pre-test of the fused frame path)
  int32_t* tile_len;     // [T] candidates per tile that the wave kernels traverse
  int32_t* counters;     // [kNumCounters]
  int64_t max_work;
  int64_t max_work_small;
  int64_t bytes;
};

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

inline int num_tiles(int W, int H, int ts) { return ((W + ts - 1) / ts) * ((H + ts - 1) / ts); }

constexpr int kScanItems = 4096;  // elements per block of the multi-block scans
constexpr int kPrimScanItems = 1024;   // primitives per block of the per-primitive scan (256 threads, four each)

// Carve the scratch block.  base may be null (size query).
inline Scratch carve_scratch(void* base, int n, int W, int H, int ts, int64_t max_pairs, int64_t max_records) {
  Scratch s;
  char* p = static_cast<char*>(base);
  int64_t off = 0;
  const int64_t T = num_tiles(W, H, ts);
  const int64_t P = (int64_t)W * H;
  auto take = [&](int64_t bytes) { char* r = p ? p + off : nullptr; off += align_up(bytes, 256); return r; };
  s.tile_cnt = (int32_t*)take(4 * (T + 1));
  s.tile_diff = (int32_t*)take(4 * (int64_t)((W + ts - 1) / ts + 1) * ((H + ts - 1) / ts + 1));
  s.tile_fill = (int32_t*)take(4 * T);
  s.rect = (uint2*)take(8 * (int64_t)n);
  const int64_t nblk = std::max<int64_t>((std::max<int64_t>(T, P + 1) + kScanItems - 1) / kScanItems,
                                         ((int64_t)n + kPrimScanItems - 1) / kPrimScanItems) + 2;
  s.scan_blk = (int32_t*)take(4 * 3 * nblk);
  s.px_state = (float4*)take(16 * P);
  s.px_depth = (float2*)take(8 * P);
  s.masks32 = (uint32_t*)take(8 * max_pairs);
  s.pair_base = (uint32_t*)take(4 * max_pairs);
  s.prim_cnt = (int32_t*)take(4 * 2 * ((int64_t)n + 4));
  s.prim_cursor = (int32_t*)take(4 * (int64_t)n);
  s.prim_off = (int32_t*)take(4 * ((int64_t)n + 1));
  s.max_work = (int64_t)n + max_records / kRowsPerItem + 2;
  s.work = (int4*)take(16 * s.max_work);
  s.max_work_small = 2 * (int64_t)n + 2;
  s.work_small = (int4*)take(16 * s.max_work_small);
  s.rec_in = (RecIn*)take(32 * max_records);
  s.rec_out = (float4*)take(16 * max_records);
  s.rec_t = (float*)take(4 * max_records);
  s.rec_gate = (float4*)take(16 * max_records);
  s.rec_w = (float*)take(4 * max_records);
  s.rec_tr = (float*)take(4 * max_records);
  s.rec_ext = (float4*)take(16 * max_records);
  s.px_cnt = (int32_t*)take(4 * (P + 2));
  s.px_off = (int32_t*)take(4 * (P + 2));
  s.used32 = (uint32_t*)take(8 * max_pairs);
  s.active[0] = (int32_t*)take(4 * T);
  s.active[1] = (int32_t*)take(4 * T);
  s.counters = (int32_t*)take(4 * kNumCounters);
  s.tile_frame = (TileFrame*)take(64 * T);
  s.tile_len = (int32_t*)take(4 * T);
  s.bytes = off;
  return s;
}

// Programmatic dependent launch.  The kernels of a frame form one dependent chain of some thirty launches; with the
// launch attribute below the next kernel of the chain is set up and its CTAs take their places while the previous
// kernel's last CTAs are still running, instead of after the previous grid has drained.  Every kernel launched this
// way begins with chain_wait(), which returns once the previous grid has completed and its writes are visible (so
// the stream's order is kept exactly), and then lets its own successor be set up (chain_release()).  On a kernel
// launched without the attribute both are no-ops.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

// Kernel classes for the launch counter and the optional per-class device timing.
enum KernelClass { kKBin = 0, kKSort, kKHits, kKScan, kKFill, kKMlp, kKComposite, kKMisc, kNumKernelClasses };

// RAII marker around the launches of one class: counts them and, when timing is enabled,
// brackets them with CUDA events on the launching stream.
struct LaunchScope {
  LaunchScope(KernelClass k, int launches, cudaStream_t st);
  ~LaunchScope();
  int slot;
  cudaStream_t st;
};

// last-error text (thread-local) for the negative return codes
void set_error(const char* fmt, ...);
int cuda_check(cudaError_t e, const char* what);

#define MLPSP_CUDA_OK(call)                                         \
  do {                                                              \
    int rc__ = ::mlpsp::cuda_check((call), #call);                  \
    if (rc__ != 0) return rc__;                                     \
  } while (0)

#define MLPSP_REQUIRE(cond, code, ...)                              \
  do {                                                              \
    if (!(cond)) { ::mlpsp::set_error(__VA_ARGS__); return (code); }\
  } while (0)

// Per-device "first use" marker for settings that CUDA keeps per device (the opt-in dynamic shared-memory
// size of a kernel, for one): a process that drives several GPUs must apply them once on each.  The caller
// keeps one DeviceOnce per setting; first() answers true the first time it is asked with a given device current.
struct DeviceOnce {
  bool seen[64] = {false};
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;   // unknown device: apply every time
    if (seen[dev]) return false;
    seen[dev] = true;
    return true;
  }
};

// stage launchers (defined in the .cu files)
// order_lists = false leaves every tile list in scatter order for a following launch_sort(unordered_input = true).
// pretest: write only the (tile, primitive) pairs that some ray of the tile can hit; s.tile_len receives the
// number kept per tile (they sit at the front of the tile's span), tile_offsets stay those of the full lists.
int launch_bin(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st, bool order_lists = true,
               bool pretest = false);
// ray frame of every 8x8 tile (TileFrame), from the frame's rays
void launch_tile_frames(const mlpsp_frame* fr, TileFrame* frames, cudaStream_t st);
int launch_bin_mosaic(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, const int32_t* tile_view,
                      const float* views_host, int num_views, cudaStream_t st);
int launch_bin_raycone(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st);
// long_list [T] / long_count [2]: device scratch (tiles that take the block-wide sort, their number, a tile cursor)
// list_len (optional): candidates actually present at the front of every tile's span (pre-tested binning);
// the rest of the span is filled with -1 in sorted_prims
int launch_sort(const mlpsp_scene* sc, const mlpsp_frame* fr, float* keys_out, cudaStream_t st, bool unordered_input,
                int32_t* long_list, int32_t* long_count, const int32_t* list_len = nullptr);
int launch_hit_masks(const mlpsp_scene* sc, const mlpsp_frame* fr, uint64_t* mask_geo, cudaStream_t st);
// lists_refined: s.tile_len already holds the traversal length of every tile (written by launch_sort)
int launch_render_sorted(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, cudaStream_t st,
                         bool lists_refined = false);
// rec_ext (optional): per record (sigma_raw, sigma_logit, layer-1 ReLU bitmask, layer-2 ReLU bitmask)
// grid_cap > 0 limits the number of CTAs (a wave that is expected to be idle)
int launch_mlp_f32(const mlpsp_scene* sc, const RecIn* rec_in, const int32_t* prim_off, const int4* work,
                   const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                   cudaStream_t st, int grid_cap = 0);
// bf16: bfloat16 operands (sc->wbf16) instead of binary16 (sc->w16)
// work_small: the wave's small-group list (launch_prim_scan with split_small), or null when every item is on `work`
// per-primitive weight gradients with binary16 / bfloat16 operands on tcgen05 (vjp_tc.cu); flag bit 1 = a wait gave up
int launch_grouped_vjp_tc(bool bf16, const float* x6, const float* d4, const int32_t* masks, const int64_t* offsets,
                          const int64_t* seg_prim, const int64_t* seg_start, int64_t num_segments, int segment_size,
                          const mlpsp_scene* sc, float scale, float* partial, int32_t* flag, cudaStream_t st);
int launch_mlp_f16(const mlpsp_scene* sc, const RecIn* rec_in, const int32_t* prim_off, const int4* work,
                   const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                   cudaStream_t st, bool bf16 = false, int grid_cap = 0, const int4* work_small = nullptr);
int launch_scan_i32(const int32_t* in, int64_t n, int32_t* blk, int32_t* out, cudaStream_t st);
int launch_export_records(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, int64_t* offsets, int32_t* ids,
                          float* x6, float* raw, int32_t* relu_masks, float* gates, int64_t max_out, int32_t max_hits,
                          int64_t* total_host, int32_t* worst_host, cudaStream_t st);

// evaluator output modes
constexpr int kOutAlpha = 0;     // (R,G,B, 1-exp(-softplus(o3)*decay)) scattered to rec.slot
constexpr int kOutSigmaRaw = 1;  // (R,G,B, softplus(o3)) scattered to rec.slot

// feature compositing on the tensor cores (feature_tc.cu): whether this scene's attributes qualify (a binary16 copy,
// 128 / 256 / 384 / 512 channels, 1, 4 or 5 slots), and the launch for a rendered frame (consumed masks in used32)
bool feature_tc_supported(const mlpsp_scene* sc);
int launch_feature_tc(const mlpsp_scene* sc, const mlpsp_frame* fr, const Scratch& s, const uint32_t* used32, cudaStream_t st);

// multi-block exclusive scan of per-primitive record counts plus evaluator work-item emission
// split_small: remainders of at most 64 records go to the small-group list (s.work_small)
// distance in elements between the count arrays of even and odd waves (keeps the second one 16-byte aligned)
__host__ __device__ inline size_t prim_cnt_stride(int n) { return ((size_t)n + 3) & ~(size_t)3; }
int launch_render_batch(const mlpsp_scene* sc, const mlpsp_frame* frs, const Scratch* ss, int V, cudaStream_t st, bool lists_refined);
int scan_launches(int64_t n);   // kernels launch_scan_i32 launches for n items
int launch_prim_scan(const Scratch& s, int n, int next_list, int32_t* status, cudaStream_t st, bool split_small = false, int wave = 0);

}  // namespace mlpsp
