/*
 * mlpsp.h - C ABI of the B200 (sm_100a) tile-centre render path of MLP Splatting.
 *
 * Drop-in boundary: these entry points stand where the reference's pybind11 extension
 * (scannet/cuda/np_tile_kernels.cu:7224-7252) and the PyTorch culling in
 * scannet/cumodel.py:994-1070 stand.  Plain pointers and sizes only; all array pointers are
 * DEVICE pointers unless a comment says "host".  Inputs are borrowed and never written; outputs
 * and scratch are allocated by the caller.  Every call is asynchronous on `stream` (a
 * cudaStream_t passed as void*) and returns 0, or a negative MLPSP_E_* code for a host-side
 * argument error (text via mlpsp_last_error()).  Device-side findings (capacity overflow, bad
 * ids, scratch too small, non-finite activations, a wait that gave up) are OR-ed into a
 * caller-owned int32 status block that the caller reads after synchronising; kernels launched
 * after a fatal finding return without touching their outputs.
 */
#ifndef MLPSP_H_
#define MLPSP_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLPSP_ABI_VERSION 1

/* host-side return codes */
#define MLPSP_OK 0
#define MLPSP_E_ARG (-1)      /* bad argument (null pointer, size, unsupported option) */
#define MLPSP_E_SCRATCH (-2)  /* scratch block smaller than mlpsp_frame_scratch_bytes() */
#define MLPSP_E_CUDA (-3)     /* a CUDA runtime call failed */
#define MLPSP_E_LIMIT (-4)    /* size beyond a documented limit */

/* status block: int32 status[MLPSP_STATUS_WORDS], zeroed by the caller or by mlpsp_status_reset */
#define MLPSP_STATUS_WORDS 16
#define MLPSP_ST_BITS 0            /* OR of the MLPSP_ST_* bits below */
#define MLPSP_ST_MAX_TILE_LEN 1    /* longest tile list seen by binning / validation */
#define MLPSP_ST_PAIRS 2           /* number of (tile, primitive) candidate pairs */
#define MLPSP_ST_WAVES 3           /* waves launched with at least one candidate window */
#define MLPSP_ST_RECORDS_LO 4      /* MLP evaluations performed this frame (64-bit, words 4-5) */
#define MLPSP_ST_RECORDS_HI 5
#define MLPSP_ST_USED_LO 6         /* records consumed by compositing (64-bit, words 6-7) */
#define MLPSP_ST_USED_HI 7
#define MLPSP_ST_WAVE_RECORDS 8    /* largest record count of a single wave */
#define MLPSP_ST_WORK_ITEMS 9      /* largest number of evaluator work items of a single wave */
#define MLPSP_ST_WORK_TOTAL 10     /* evaluator work items (blocks of at most 128 rows) of the whole frame */
#define MLPSP_ST_PAIRS_KEPT 11     /* mlpsp_render_frame: candidate pairs left after the tile pre-test */
#define MLPSP_ST_WORK_SMALL 12     /* of MLPSP_ST_WORK_TOTAL: items of the small-group list (at most 32 rows) */

/* bits 1,2,4 match the reference validator (np_tile_kernels.cu:4499-4519) */
#define MLPSP_ST_BAD_OFFSETS 1       /* tile_offsets not 0-based / monotone / in bounds */
#define MLPSP_ST_TILE_CAPACITY 2     /* a tile list is longer than tile_capacity */
#define MLPSP_ST_BAD_IDS 4           /* candidate id outside [0, n) */
#define MLPSP_ST_PAIR_OVERFLOW 8     /* more candidate pairs than max_pairs */
#define MLPSP_ST_RECORD_OVERFLOW 16  /* a wave produced more records than max_records */
#define MLPSP_ST_PIXEL_HITS 32       /* per-pixel ordering: a pixel met more than 256 primitives */
#define MLPSP_ST_NUMERIC 64          /* non-finite operand/activation in the fp16 evaluator */
#define MLPSP_ST_TIMEOUT 128         /* a bounded device-side wait gave up */
#define MLPSP_ST_TILE_ORIGINS 256    /* ray-cone culling: a tile's rays do not share one origin */
#define MLPSP_ST_CONE_TOO_WIDE 512   /* ray-cone culling: a tile's ray cone spans >= 90 degrees */
#define MLPSP_ST_FEAT_INEXACT 1024   /* mlpsp_pack_features_f16: an attribute is not representable in binary16 */
#define MLPSP_ST_FATAL (1 | 2 | 4 | 8 | 16 | 128 | 256 | 512)

#define MLPSP_PRECISION_F32 0  /* scalar FP32 evaluator (np_tile_kernels.cu:312-380) */
#define MLPSP_PRECISION_F16 1  /* fp16 operands, FP32 accumulate, tcgen05 (rgb_wmma.cuh:75-223) */
#define MLPSP_PRECISION_BF16 2 /* bfloat16 operands (the bf16 flag of render_tiles_rgb_wmma, rgb_wmma.cuh:225), same kernel */
#define MLPSP_ORDER_PER_PIXEL 2 /* value of mlpsp_frame.sort_key for per-pixel exact ordering */

#define MLPSP_GEOM_FLOATS 16   /* packed geometry floats per primitive */
#define MLPSP_MAX_WAVES 32

/* Scene parameters (borrowed).  Replaces the 15-tensor argument list of the reference entry
 * points (np_tile_kernels.cu:5225-5247): positions/log_scales/quats arrive packed by
 * mlpsp_pack_geometry; W1..b3, freq, att keep the reference layouts
 * (W1[n,H,12F], b1[n,H], W2[n,H,H], b2[n,H], W3[n,4,H], b3[n,4], row-major FP32). */
typedef struct mlpsp_scene {
  const float* geom;      /* [n*16] from mlpsp_pack_geometry */
  int32_t n;
  int32_t hidden;         /* H <= 64 (FP32 evaluator), 32 or 64 (fp16 / bf16 tensor-core evaluator) */
  int32_t num_freq;       /* F <= 8; encoded width IN = 12 F; fp16 evaluator needs F == 6 */
  int32_t reserved0;
  const float* W1; const float* b1; const float* W2; const float* b2; const float* W3; const float* b3;
  const void* w16;        /* [n * mlpsp_packed_weight_bytes()] from mlpsp_pack_weights_f16, or NULL */
  const float* freq;      /* [F] */
  const float* att;       /* [F] */
  const float* feat_attr; /* [n, feat_slots, feat_dim] or NULL */
  int32_t feat_slots;     /* 1, 4 or 5 (np_tile_kernels.cu:6036-6075) */
  int32_t feat_dim;       /* C <= 512 */
  float gate_beta;        /* semantic_tetra_gates norm_beta */
  float gate_tau;         /* semantic_tetra_gates logit_temp */
  const void* wbf16;      /* the same image with bfloat16 operands, from mlpsp_pack_weights_bf16, or NULL */
  const void* feat16;     /* feat_attr as binary16 [n, feat_slots, feat_dim] from mlpsp_pack_features_f16, or NULL.  When
                             set, and feat_dim is 128, 256, 384 or 512, the feature map is composited on the tensor
                             cores from this copy (FP32 accumulation); otherwise from feat_attr on the FP32 path. */
} mlpsp_scene;

/* One frame.  Replaces (rays_o, rays_d, culled_prim_indices, tile_offsets, Wimg, Himg, TW, TH,
 * threshold) of the reference entry points plus their freshly allocated outputs. */
typedef struct mlpsp_frame {
  const float* rays_o;    /* [W*H,3] */
  const float* rays_d;    /* [W*H,3], unit length (the reference passes F.normalize(ray_d)) */
  int32_t width, height;
  int32_t tile;           /* 8 */
  float threshold;        /* score threshold in (0,1) */
  int32_t tile_capacity;  /* 1536 (MLPSP_MAX_TILE_PRIMS of the reference loader) */
  int32_t precision;      /* MLPSP_PRECISION_* */
  const float* view;      /* HOST [16] row-major view matrix (binning only) */
  const float* proj;      /* HOST [16] row-major projection matrix (binning only) */
  int32_t* tile_offsets;  /* [T+1]  written by binning, read by the later stages */
  int32_t* tile_prims;    /* [max_pairs] candidate ids, ascending inside a tile */
  int32_t* sorted_prims;  /* [max_pairs] the same lists in tile-centre depth order */
  int64_t max_pairs;
  float* rgb;             /* [W*H,3] */
  float* alpha;           /* [W*H]   */
  float* depth_t;         /* [W*H] expected depth sum(w t)/sum(w), or NULL */
  float* feat;            /* [W*H, feat_dim] composited features, or NULL */
  uint64_t* mask_used;    /* [max_pairs] per pair: pixels (bit = ly*8+lx) whose record was composited, or NULL */
  const float* bg_color;  /* HOST [3] background added as rgb + clamp(1-alpha,0,1)*bg, or NULL */
  void* scratch;          /* mlpsp_frame_scratch_bytes() bytes, 256-byte aligned */
  int64_t scratch_bytes;
  int64_t max_records;    /* record capacity of one wave */
  int32_t* status;        /* [MLPSP_STATUS_WORDS] */
  int32_t num_waves;      /* 0 = library default schedule */
  int32_t wave_len[MLPSP_MAX_WAVES]; /* candidates per tile processed by wave k */
  int32_t keep_records;   /* 1 = keep what mlpsp_export_records needs (ReLU masks, logits, transmittance) */
  int32_t sort_key;       /* 0 = t* of the tile-centre ray (np_tile_kernels.cu:483-518), the order of the forward,
                             feature and record kernels; 1 = Euclidean depth (c - o).d along that ray, the order
                             of render_tiles_kernel_tilecenter_order_with_t (np_tile_kernels.cu:5538-5543);
                             2 (MLPSP_ORDER_PER_PIXEL) = per-pixel exact ordering, render_tiles_kernel_with_sort
                             (np_tile_kernels.cu:714-926): every pixel blends its own hits in the order of its own
                             hit distances; rgb, alpha and the feature map only, every hit is evaluated (size max_records for all
                             hits of the frame), more than 256 hits in a pixel raise MLPSP_ST_PIXEL_HITS */
  int32_t tile_row_begin; /* binning keeps only tile rows [tile_row_begin, tile_row_end); both 0 = the whole image. */
  int32_t tile_row_end;   /* Used to share one view between GPUs by bands of tile rows: tiles outside the band get
                             empty lists and their pixels the background. */
  int32_t tile_pretest;   /* mlpsp_render_frame only.  0 = while binning, drop every candidate that no ray of its
                             tile can hit (a conservative ellipsoid-against-tile test with no reference
                             counterpart; the image is the same, the lists the wave kernels walk are shorter);
                             it is skipped when mask_used is requested, so that those masks stay aligned with the
                             full sorted lists.  1 = never drop.  With the test on, sorted_prims holds the kept
                             candidates of every tile in depth order followed by -1 entries. */
  int32_t tail_hint;      /* 1 = the last wave is expected to find no work (a host that carries the wave schedule
                             from frame to frame knows): its kernels are launched with one CTA per SM instead of
                             full grids.  Whatever work it does find is still done; only its speed changes. */
  /* Per-primitive contribution statistics of render_tiles_kernel_tilecenter_stats (np_tile_kernels.cu:2143-2500),
   * all NULL or all set; the five [n] arrays are accumulated into, never reset.  With w = trans * alpha of a
   * composited record: sum_w += w; max_w = max(max_w, w); hits += (w > 1e-8); for w > 0.1: contrib += 1 and
   * sum_werr += w * L1(colour after this record - gt_rgb). */
  const float* gt_rgb;    /* [width*height, 3] */
  float* stat_sum_w;
  float* stat_max_w;
  int32_t* stat_hits;
  float* stat_sum_werr;
  int32_t* stat_contrib;
  int32_t hit_arith;      /* arithmetic of the tile-centre key, the hit decision and the hit values: 0 = IEEE-only
                             operations in a fixed order with a software exponential, which a CPU reproduces bit for bit
                             (tile lists, order and masks are then exactly the CPU restatement's); 1 = the reference
                             kernels' own arithmetic (hardware __expf, compiler-contracted expressions,
                             np_tile_kernels.cu:416-435, 483-518, 659-711), which makes order, masks, record lists and
                             CSR offsets those of the reference's kernels run on the same GPU.  The images of the two
                             differ only where a value lies within a few ulp of a threshold. */
  int32_t reserved1;
} mlpsp_frame;

const char* mlpsp_last_error(void);
int mlpsp_abi_version(void);
/* sizeof(mlpsp_scene), sizeof(mlpsp_frame) as compiled, for bindings that mirror the structs */
int mlpsp_struct_sizes(int32_t* scene_bytes, int32_t* frame_bytes);

/* positions[n,3], log_scales[n,3], unit quats[n,4] -> geom[n*16]
 * (the per-primitive loads of np_tile_kernels.cu:1948-1957, with exp(-2 ls) hoisted) */
int mlpsp_pack_geometry(const float* positions, const float* log_scales, const float* quats_unit,
                        int32_t n, float* geom, void* stream);

/* out = in / max(|in|, 1e-12) per row of `dim` (3 or 4) floats: F.normalize at cumodel.py:1088,1114 */
int mlpsp_normalize_rows(const float* in, float* out, int64_t rows, int32_t dim, void* stream);

/* Bytes per primitive of the fp16 evaluator's packed weight image, and the packer.  Replaces the
 * per-(tile, primitive) FP32->fp16 re-cast of rgb_wmma.cuh:162-176 with one cast per scene. */
int64_t mlpsp_packed_weight_bytes(int32_t hidden, int32_t num_freq);
/* status (optional): MLPSP_ST_NUMERIC is raised when a weight or bias is not finite in fp16/FP32. */
int mlpsp_pack_weights_f16(const mlpsp_scene* scene, void* w16_out, int32_t* status, void* stream);
/* The same image with bfloat16 operands (same size and layout); no reference kernel casts per scene either. */
int mlpsp_pack_weights_bf16(const mlpsp_scene* scene, void* wbf16_out, int32_t* status, void* stream);

/* binary16 copy of scene->feat_attr [n, feat_slots, feat_dim] (the storage format of the reference's inference
 * export, scannet/checkpoints.py:358-359) for the tensor-core feature compositing.  status (optional):
 * MLPSP_ST_FEAT_INEXACT is raised when some attribute does not survive the round trip, i.e. when rendering from
 * the copy would differ from rendering from feat_attr by binary16 rounding of the attributes. */
int mlpsp_pack_features_f16(const mlpsp_scene* scene, void* feat16_out, int32_t* status, void* stream);

int mlpsp_status_reset(int32_t* status, void* stream);

/* Launch accounting.  Kernel classes: 0 bin, 1 sort, 2 hit pass, 3 per-primitive scan, 4 record fill,
 * 5 evaluator, 6 compositing, 7 other.  mlpsp_kernel_launches returns the number of kernels this
 * library has launched in the process (per class in per_class[0..num_classes), optional).
 * With timing enabled every launch group is bracketed by CUDA events on its stream;
 * mlpsp_timing_collect waits for them, adds the elapsed milliseconds per class into
 * ms_per_class[MLPSP_KERNEL_CLASSES] and forgets them.  Not thread-safe; meant for benchmarks. */
#define MLPSP_KERNEL_CLASSES 8
int mlpsp_kernel_launches(int64_t* per_class, int32_t num_classes);
int mlpsp_timing_enable(int32_t on);
int mlpsp_timing_collect(float* ms_per_class, int32_t num_classes);

/* Scratch size for a frame of this shape. */
int64_t mlpsp_frame_scratch_bytes(int32_t n, int32_t width, int32_t height, int32_t tile,
                                  int64_t max_pairs, int64_t max_records);

/* Screen-space culling: cumodel.py:994-1070 (overlap predicate, tile-major lists, ascending id).
 * Writes frame->tile_offsets, frame->tile_prims; status words 1,2 and bits 2,8.
 * frame->tile may be 8 or 16 here and in mlpsp_sort_tiles (the reference's tile_size = 16: culling, capacity and
 * tile-centre order per 16x16 tile); every other entry point works on 8x8 tiles, and a 16x16 frame is rendered by
 * giving each 8x8 tile the ordered list of its 16x16 tile (pre-sorted lists into mlpsp_render_sorted). */
int mlpsp_bin_tiles(const mlpsp_scene* scene, const mlpsp_frame* frame, void* stream);

/* Culling for mosaic frames whose tiles come from different views
 * (build_tilecenter_culling_from_tile_views, cumodel.py:838-949): tile t uses view tile_view_ids[t]
 * (device int32[T], values in [0, num_views)); view_matrices is HOST [num_views*16] row-major;
 * frame->proj is shared by all views, frame->view is ignored. */
int mlpsp_bin_tiles_mosaic(const mlpsp_scene* scene, const mlpsp_frame* frame, const int32_t* tile_view_ids,
                           const float* view_matrices, int32_t num_views, void* stream);

/* Conservative culling from the actual rays, for cameras a projection matrix cannot describe
 * (ray_cone_candidates, scannet/camera.py:102-146): per tile the cone around its 64 rays (pixels
 * clamped to the image), per primitive its enclosing sphere of radius max scale * sqrt(-2 ln thr);
 * a primitive is kept when the sphere touches the cone.  Reads frame->rays_o and frame->rays_d (any
 * length; normalised inside), writes frame->tile_offsets / tile_prims (ascending id). */
int mlpsp_bin_tiles_raycone(const mlpsp_scene* scene, const mlpsp_frame* frame, void* stream);

/* validate_tile_candidate_capacity (np_tile_kernels.cu:4485-4589) for caller-supplied lists of
 * `pairs` candidates. */
int mlpsp_validate_tile_lists(const int32_t* tile_offsets, const int32_t* tile_prims, int32_t num_tiles,
                              int64_t pairs, int32_t tile_capacity, int32_t n, int32_t* status,
                              void* stream);

/* Per-tile stable ascending sort by the tile-centre key (np_tile_kernels.cu:483-518, 1914-1990).
 * Reads tile_offsets/tile_prims, writes sorted_prims; keys_out ([max_pairs], optional) receives
 * the sorted keys. */
int mlpsp_sort_tiles(const mlpsp_scene* scene, const mlpsp_frame* frame, float* keys_out, void* stream);

/* Geometric hit mask of every pair of the sorted lists, no termination
 * (hit_and_features_rot, np_tile_kernels.cu:659-711): mask_geo[pair] bit ly*8+lx. */
int mlpsp_hit_masks(const mlpsp_scene* scene, const mlpsp_frame* frame, uint64_t* mask_geo, void* stream);

/* Records -> per-primitive evaluation -> compositing for depth-sorted lists: the body of
 * render_tiles_kernel_tilecenter_order (np_tile_kernels.cu:1837-2137), render_rgb_wmma_kernel
 * (rgb_wmma.cuh:75-223), ..._with_t (5432-5718) and ..._with_feat (5794-6112). */
int mlpsp_render_sorted(const mlpsp_scene* scene, const mlpsp_frame* frame, void* stream);

/* bin + sort + render_sorted: what NeuralPrimitiveSceneTileCUDA.forward does per frame
 * (cumodel.py:951-1160).  Here frame->tile_prims is left in binning scatter order (the per-tile sort
 * breaks depth ties by id, which gives the same sorted_prims as sorting the ascending-id lists);
 * call mlpsp_bin_tiles when the ascending-id lists themselves are wanted.  See frame->tile_pretest for
 * what sorted_prims holds afterwards. */
int mlpsp_render_frame(const mlpsp_scene* scene, const mlpsp_frame* frame, void* stream);

/* Several views of one scene in one call (no reference counterpart: the reference renders view by view,
 * scannet/cumodel.py:951).  frames[0..num_frames) are complete frames as for mlpsp_render_frame -- own rays,
 * matrices, tile-list buffers, outputs and scratch block each -- of one shape, threshold, precision, tile
 * capacity and hit_arith, rgb and alpha only (no depth, features, masks, records, statistics, bands), and they
 * share ONE status block (frames[v].status == frames[0].status; its words are then sums / maxima over the views,
 * and an error bit of any view fails the batch).  Binning, sorting, hit masks, record fill and compositing run per
 * view; the per-primitive record counts, CSR offsets, work list and record arrays are those of frames[0]'s
 * scratch, so frames[0].max_records must cover the MLP evaluations of ALL views (the other frames may be sized
 * with max_records = 0) and one evaluator launch per wave serves every view: a primitive's weights are fetched
 * once per wave instead of once per wave and view.  Images are bit-identical to frames rendered alone. */
#define MLPSP_MAX_BATCH 64
int mlpsp_render_frames(const mlpsp_scene* scene, const mlpsp_frame* frames, int32_t num_frames, void* stream);

/* Pixel-major records of the frame just rendered with frame->keep_records = 1 on the same scratch: the
 * 8-tensor schema of render_tiles_training_records (np_tile_kernels.cu:3138-3154, 6897-6986;
 * training_wmma.cuh:223-256).  Records of a pixel are in compositing order and hold only the hits that
 * were composited.  offsets[W*H+1] int64 is always written and *total_host receives the record count
 * (the call synchronises).  ids[R] int32, x6[R,6], raw[R,8] = (R,G,B,sigma_raw,trans_before,alpha,decay,
 * sigma_logit), relu_masks[R,2] int32, gates[R,4] are written when non-NULL and max_out >= R.
 * max_hits: per-pixel record capacity (512 in the reference build); *worst_host receives the largest
 * per-pixel count, negated when a pixel reached the capacity while still live (the reference's
 * "hit capacity" error). */
int mlpsp_export_records(const mlpsp_scene* scene, const mlpsp_frame* frame, int64_t* offsets, int32_t* ids,
                         float* x6, float* raw, int32_t* relu_masks, float* gates, int64_t max_out,
                         int32_t max_hits, int64_t* total_host, int32_t* worst_host, void* stream);

/* Grouped evaluator on explicit records (the forward counterpart of primitive_gemm.py's grouped
 * VJP): records are primitive-major, offsets[n+1] int64 as produced by group_records
 * (primitive_csr.py:23-29); x6[R,6]; out[R,4] = (R, G, B, sigma_raw). */
int64_t mlpsp_mlp_grouped_scratch_bytes(int64_t num_records, int32_t n);
int mlpsp_mlp_grouped(const mlpsp_scene* scene, int32_t precision, const int64_t* offsets, const float* x6,
                      int64_t num_records, float* out4, void* scratch, int64_t scratch_bytes,
                      int32_t* status, void* stream);

/* group_records (primitive_csr.py:23-29): stable grouping of R record ids by primitive.
 * offsets[n+1] int64, order[R] int64 (record indices, ascending inside a group). */
int64_t mlpsp_group_records_scratch_bytes(int64_t num_records, int32_t n);
int mlpsp_group_records(const int32_t* primitive_ids, int64_t num_records, int32_t n, int64_t* offsets,
                        int64_t* order, void* scratch, int64_t scratch_bytes, void* stream);

/* prepare_groups (primitive_gemm.py:186-203): split every primitive's records into segments of at
 * most segment_size.  group_offsets[n+1] int64 is always written; of primitives/starts ([G] int64, may be
 * NULL) the first min(G, max_groups) entries are written, so a caller may ask for G first (max_groups = 0)
 * and call again.  *num_groups_host receives G (the call synchronises).  More than 2^31-1 groups in total
 * are rejected with MLPSP_E_LIMIT (the outputs are then undefined). */
int mlpsp_prepare_groups(const int64_t* offsets, int32_t n, int64_t segment_size, int64_t* group_offsets,
                         int64_t* primitives, int64_t* starts, int64_t max_groups,
                         int64_t* num_groups_host, void* stream);

/* prepare_groups for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Same arguments and results as mlpsp_prepare_groups, but it calls no cudaMalloc/cudaFree:
 * its work arrays live in a fixed device array inside the library (about 4 MiB on every GPU that loads
 * the library, until the process exits), which limits it to n <= MLPSP_STATIC_GROUPS_MAX_PRIMITIVES;
 * larger n is rejected with MLPSP_E_LIMIT.  Meant for hosts whose embedding application owns all device
 * memory and forbids allocations after start-up, or whose frame loop must avoid the device-wide
 * synchronisation of cudaMalloc/cudaFree.  The first call on each device looks up the array's device
 * address, so issue that first call outside any stream capture.  All calls share the array: calls that
 * overlap on the GPU race on it, so keep them on one stream or otherwise serialised. */
#define MLPSP_STATIC_GROUPS_MAX_PRIMITIVES 524288
int mlpsp_prepare_groups_static(const int64_t* offsets, int32_t n, int64_t segment_size, int64_t* group_offsets,
                                int64_t* primitives, int64_t* starts, int64_t max_groups,
                                int64_t* num_groups_host, void* stream);

/* ---- backward side of the record path (training callers) ---- */

/* Reverse compositing over saved records: primitive_records_reverse (scannet/cuda/primitive_records.cuh:3-74).
 * ids[R], offsets[pixels+1] (int64, pixel-major records in compositing order), x6[R,6], raw[R,8] as written by
 * mlpsp_export_records; log_scales[n,3], quats[n,4] (unit); grad_rgb[pixels,3], grad_t[pixels] (adjoint of the
 * final transmittance); total_records = R = offsets[pixels].  Writes d4[R,4] (adjoints of the four pre-activation
 * MLP outputs) and the position / log-scale / quaternion gradients [n,3] [n,3] [n,4], which are zeroed first.
 * raw, d4 and quats must be 16-byte aligned. */
int mlpsp_records_reverse(const int32_t* ids, const int64_t* offsets, const float* x6, const float* raw,
                          const float* log_scales, const float* quats, const float* grad_rgb, const float* grad_t,
                          int64_t pixels, int64_t total_records, int32_t n, float* d4, float* grad_pos,
                          float* grad_log_scales, float* grad_quats, void* stream);

/* Floats per primitive of the packed gradient row: W1[32,72] b1[32] W2[32,32] b2[32] W3[4,32] b3[4] = 3,524. */
int64_t mlpsp_grouped_gradient_floats(void);

/* Per-primitive MLP weight gradients from primitive-major records: one launch of grouped_weight_gradients
 * (scannet/primitive_gemm.py:101-232; the PyTorch statement is scannet/primitive_csr.py:33-58).
 * offsets[n+1] / x6[R,6] / d4[R,4] / relu_masks[R,2] (or NULL: signs are recomputed) are a PrimitiveCSR; seg_prim,
 * seg_start [G] and seg_offsets [n+1] are a prepared group layout (mlpsp_prepare_groups) with segment_size records
 * per segment.  partial [G, 3524] is scratch; result [n, 3524].
 * precision: MLPSP_PRECISION_F32 = IEEE FP32 on the CUDA cores (the reference's float32 mode, no TF32);
 * MLPSP_PRECISION_F16 / _BF16 = operands rounded to binary16 / bfloat16, products on the tensor cores (tcgen05),
 * FP32 accumulation over the whole segment (the reference's tl.dot modes); d4 must then be 16-byte aligned.
 * loss_scale multiplies the adjoints before the cast and divides the sums after (the reference uses 4096 for
 * binary16, 1 otherwise).  *nonfinite: bit 0 = a sum is not finite -- the caller retries a mixed-precision call
 * with MLPSP_PRECISION_F32 and loss_scale 1 as primitive_gemm.py:64-98 does (the host mirror does);
 * bit 1 = a device-side wait gave up, results invalid. */
int mlpsp_grouped_weight_gradients(const mlpsp_scene* scene, const int64_t* offsets, const float* x6, const float* d4,
                                   const int32_t* relu_masks, const int64_t* seg_prim, const int64_t* seg_start,
                                   const int64_t* seg_offsets, int64_t num_segments, int32_t segment_size,
                                   int32_t precision, float loss_scale, float* partial, float* result,
                                   int32_t* nonfinite, void* stream);

/* ---- the step after the feature map: feature decoder and text query ---- */

/* The reference's FeatureUpsampleDecoder (scannet/feature_decoder.py:5-19): conv 1x1 -> ReLU -> conv 3x3 (zero
 * padding 1) -> ReLU -> conv 1x1, weights in torch Conv2d layout (device pointers, FP32):
 * W1 [hidden, in_dim] (net.0), W2 [hidden, hidden, 3, 3] (net.2), W3 [out_dim, hidden] (net.4).
 * text [num_classes, out_dim] are the (unnormalised) text embeddings of a query, or NULL. */
typedef struct mlpsp_decoder {
  int32_t in_dim, hidden, out_dim, num_classes;
  const float *W1, *b1, *W2, *b2, *W3, *b3;
  const float* text;
} mlpsp_decoder;

/* Bytes of the packed binary16 image of a decoder (0: sizes outside the limits: in_dim <= 128, hidden 32 / 64 /
 * 96 / 128, at most 768 outputs or classes).  mode 0: the image computes the decoded features; mode 1: the last
 * layer is folded with the normalised text embeddings (text^ W3, text^ b3) and the image computes class scores. */
int64_t mlpsp_decoder_packed_bytes(const mlpsp_decoder* dec, int32_t mode);
int mlpsp_pack_decoder(const mlpsp_decoder* dec, int32_t mode, void* packed, int32_t* status, void* stream);

/* Run the decoder over a pixel-major feature map feat [height*width, in_dim] (what mlpsp_render_frame writes into
 * frame.feat) on the tensor cores: binary16 operands, FP32 accumulation, FP32 bias (the contract of the
 * tensor-core MLP).  mode 0 writes out [height*width, out_dim] = decoder(feat) (feature_decoder.py:18-19 with the
 * permutes of eval_lseg_table2.py:1221-1225 folded away); mode 1 writes labels [height*width] (int64) =
 * _classify_feature_map(decoder(feat), text) (eval_lseg_table2.py:622-641) without forming the wide map.
 * Inputs or activations beyond binary16 range raise MLPSP_ST_NUMERIC in status. */
int mlpsp_decode_features(const mlpsp_decoder* dec, int32_t mode, const void* packed, const float* feat,
                          int32_t width, int32_t height, float* out, int64_t* labels, int32_t* status, void* stream);

/* Text query of a full-width feature map in FP32: _classify_feature_map (eval_lseg_table2.py:622-641), for scenes
 * whose rendered feature already has the text embedding's width (no decoder, eval_lseg_table2.py:754-755).
 * feat [pixels, dim], text [num_classes, dim], labels [pixels] (int64); dim <= 1024, num_classes <= 1024. */
int mlpsp_classify_features(const float* feat, int64_t pixels, int32_t dim, const float* text, int32_t num_classes,
                            int64_t* labels, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MLPSP_H_ */
