"""Host side of the render path: device-resident packed scenes, per-frame scratch, status handling.

PyTorch is used for device memory, streams and the host<->device copies; every computation goes
through the C ABI of libmlpsp_b200.so (see _lib.py).  Error texts follow the reference's
TORCH_CHECK messages (scannet/cuda/np_tile_kernels.cu:4578-4588) so callers' tests can match them.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib as L

TILE = 8
TILE_CAPACITY = 1536  # MLPSP_TILE_CANDIDATE_CAPACITY default of the reference loader (cumodel.py:102-104)


def _stream_ptr(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _dev_f32(x, device):
    t = torch.as_tensor(x)
    return t.to(device=device, dtype=torch.float32).contiguous()


def normalize_rows(x: torch.Tensor) -> torch.Tensor:
    """x / max(|x|, 1e-12) per row (rows of 3 or 4 floats) on the tensor's CUDA device."""
    lib = L.load()
    x = x.contiguous().float()
    out = torch.empty_like(x)
    L.check(lib.mlpsp_normalize_rows(L.ptr(x), L.ptr(out), x.shape[0], x.shape[1], _stream_ptr(x.device)),
            "mlpsp_normalize_rows")
    return out


class PackedScene:
    """Scene parameters resident on one GPU in the layouts the kernels read.

    Takes the reference's parameter tensors (cumodel.py:724-743): positions[n,3], log_scales[n,3],
    quats[n,4] (any norm), W1[n,H,12F], b1[n,H], W2[n,H,H], b2[n,H], W3[n,4,H], b3[n,4], freq[F],
    att[F] and optionally feat_attr[n,S,C].
    """

    def __init__(self, positions, log_scales, quats, W1, b1, W2, b2, W3, b3, freq, att, feat_attr=None,
                 gate_beta=1.5, gate_tau=2.0, device="cuda", pack_f16=True, pack_bf16=False, feat_f16="exact"):
        """feat_f16: "exact" keeps a binary16 copy of feat_attr for the tensor-core feature compositing when every
        attribute is representable in binary16 (the reference's inference export stores them so,
        scannet/checkpoints.py:358-359), "round" keeps it even when the copy rounds, "off" never."""
        lib = L.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("PackedScene must live on a CUDA device; there is no CPU path")
        d = self.device
        with torch.cuda.device(d):
            self.positions = _dev_f32(positions, d)
            self.log_scales = _dev_f32(log_scales, d)
            self.quats_unit = normalize_rows(_dev_f32(quats, d))
            self.W1, self.b1, self.W2 = _dev_f32(W1, d), _dev_f32(b1, d), _dev_f32(W2, d)
            self.b2, self.W3, self.b3 = _dev_f32(b2, d), _dev_f32(W3, d), _dev_f32(b3, d)
            self.freq, self.att = _dev_f32(freq, d), _dev_f32(att, d)
            self.n = int(self.positions.shape[0])
            self.hidden = int(self.W1.shape[1]) if self.n else 32
            self.num_freq = int(self.freq.numel())
            if self.n and int(self.W1.shape[2]) != 12 * self.num_freq:
                raise ValueError("W1 input width must be 12 * num_frequencies")
            self.geom = torch.empty((max(self.n, 1), L.GEOM_FLOATS), device=d, dtype=torch.float32)
            L.check(lib.mlpsp_pack_geometry(L.ptr(self.positions), L.ptr(self.log_scales), L.ptr(self.quats_unit),
                                            self.n, L.ptr(self.geom), _stream_ptr(d)), "mlpsp_pack_geometry")
            self.feat_attr = None
            self.feat_slots, self.feat_dim = 0, 0
            if feat_attr is not None:
                fa = _dev_f32(feat_attr, d)
                if fa.dim() == 2:
                    fa = fa[:, None, :].contiguous()
                self.feat_attr, self.feat_slots, self.feat_dim = fa, int(fa.shape[1]), int(fa.shape[2])
            self.gate_beta, self.gate_tau = float(gate_beta), float(gate_tau)
            self.w16 = None
            self.wbf16 = None
            self.feat16 = None
            self.f16_rejected = False
            self.c = self._struct()
            self._pack_features(feat_f16)
            wbytes = int(lib.mlpsp_packed_weight_bytes(self.hidden, self.num_freq))
            if pack_f16 and wbytes > 0 and self.n > 0:
                w16 = torch.empty(self.n * wbytes, device=d, dtype=torch.uint8)
                st = torch.zeros(L.STATUS_WORDS, device=d, dtype=torch.int32)
                L.check(lib.mlpsp_pack_weights_f16(C.byref(self.c), L.ptr(w16), L.ptr(st), _stream_ptr(d)),
                        "mlpsp_pack_weights_f16")
                # weights that are not finite in binary16 keep the scene on the FP32 evaluator, which is
                # what the reference's per-frame overflow check amounts to (rgb_wmma.cuh:162-176, 260-272)
                if int(st[L.ST_BITS].item()) & L.BIT_NUMERIC:
                    self.f16_rejected = True
                else:
                    self.w16 = w16
                self.c = self._struct()
            if pack_bf16 and wbytes > 0 and self.n > 0:
                # the same image with bfloat16 operands (the bf16 flag of render_tiles_rgb_wmma, rgb_wmma.cuh:225)
                wb = torch.empty(self.n * wbytes, device=d, dtype=torch.uint8)
                st = torch.zeros(L.STATUS_WORDS, device=d, dtype=torch.int32)
                L.check(lib.mlpsp_pack_weights_bf16(C.byref(self.c), L.ptr(wb), L.ptr(st), _stream_ptr(d)),
                        "mlpsp_pack_weights_bf16")
                if not (int(st[L.ST_BITS].item()) & L.BIT_NUMERIC):
                    self.wbf16 = wb
                self.c = self._struct()

    @classmethod
    def from_packed_image(cls, positions, log_scales, quats, freq, att, w16, hidden, feat_attr=None, gate_beta=1.5,
                          gate_tau=2.0, device="cuda"):
        """A scene that holds geometry and an already packed fp16 weight image (mlpsp_pack_weights_f16, biases
        included) but no FP32 weight masters: it renders on the tensor-core evaluator only, and a frame that
        overflows binary16 cannot be rendered again in FP32."""
        lib = L.load()
        self = cls.__new__(cls)
        self.device = d = torch.device(device)
        if d.type != "cuda":
            raise RuntimeError("PackedScene must live on a CUDA device; there is no CPU path")
        with torch.cuda.device(d):
            self.positions, self.log_scales = _dev_f32(positions, d), _dev_f32(log_scales, d)
            self.quats_unit = normalize_rows(_dev_f32(quats, d))
            self.W1 = self.b1 = self.W2 = self.b2 = self.W3 = self.b3 = None
            self.freq, self.att = _dev_f32(freq, d), _dev_f32(att, d)
            self.n, self.hidden, self.num_freq = int(self.positions.shape[0]), int(hidden), int(self.freq.numel())
            if int(w16.numel()) != self.n * int(lib.mlpsp_packed_weight_bytes(self.hidden, self.num_freq)):
                raise ValueError("weight image size does not match the primitive count and hidden width")
            self.geom = torch.empty((max(self.n, 1), L.GEOM_FLOATS), device=d, dtype=torch.float32)
            L.check(lib.mlpsp_pack_geometry(L.ptr(self.positions), L.ptr(self.log_scales), L.ptr(self.quats_unit),
                                            self.n, L.ptr(self.geom), _stream_ptr(d)), "mlpsp_pack_geometry")
            self.feat_attr, self.feat_slots, self.feat_dim = None, 0, 0
            if feat_attr is not None:
                fa = _dev_f32(feat_attr, d)
                if fa.dim() == 2:
                    fa = fa[:, None, :].contiguous()
                self.feat_attr, self.feat_slots, self.feat_dim = fa, int(fa.shape[1]), int(fa.shape[2])
            self.gate_beta, self.gate_tau = float(gate_beta), float(gate_tau)
            self.w16, self.wbf16, self.f16_rejected = w16, None, False
            self.feat16 = None
            self.c = self._struct()
            self._pack_features("exact")
        return self

    def _pack_features(self, mode):
        """binary16 copy of feat_attr for the tensor-core feature compositing (see __init__)."""
        self.feat16 = None
        if self.feat_attr is None or mode == "off" or self.n == 0:
            return
        if mode not in ("exact", "round"):
            raise ValueError("feat_f16 must be 'exact', 'round' or 'off'")
        lib, d = L.load(), self.device
        f16 = torch.empty(self.feat_attr.shape, device=d, dtype=torch.float16)
        st = torch.zeros(L.STATUS_WORDS, device=d, dtype=torch.int32)
        L.check(lib.mlpsp_pack_features_f16(C.byref(self.c), L.ptr(f16), L.ptr(st), _stream_ptr(d)), "mlpsp_pack_features_f16")
        if mode == "round" or not (int(st[L.ST_BITS].item()) & L.BIT_FEAT_INEXACT):
            self.feat16 = f16
        self.c = self._struct()

    def _struct(self) -> L.Scene:
        s = L.Scene()
        s.geom, s.n, s.hidden, s.num_freq = L.ptr(self.geom), self.n, self.hidden, self.num_freq
        s.W1, s.b1, s.W2, s.b2, s.W3, s.b3 = (L.ptr(t) for t in (self.W1, self.b1, self.W2, self.b2, self.W3, self.b3))
        s.w16 = L.ptr(self.w16)
        s.wbf16 = L.ptr(self.wbf16)
        s.feat16 = L.ptr(getattr(self, "feat16", None))
        s.freq, s.att = L.ptr(self.freq), L.ptr(self.att)
        s.feat_attr, s.feat_slots, s.feat_dim = L.ptr(self.feat_attr), self.feat_slots, self.feat_dim
        s.gate_beta, s.gate_tau = self.gate_beta, self.gate_tau
        return s

    def with_text_query(self, text_feature) -> "PackedScene":
        """A view of this scene whose per-primitive features are projected onto the normalised text embeddings
        text_feature [C, feat_dim]: feat_attr' = feat_attr . text^T, [n, S, C].  Compositing is linear in the
        features, so the feature map rendered from the view is the map of class scores f . t^_c, and its
        per-pixel arg-max equals _classify_feature_map on the full-width map (scannet/eval_lseg_table2.py:622-641;
        the per-pixel normalisation there is one positive factor).  Geometry and MLP weights are shared."""
        import copy
        if self.feat_attr is None:
            raise RuntimeError("Scene has no semantic feature branch (feat_attr).")
        t = _dev_f32(text_feature, self.device)
        if t.ndim != 2 or int(t.shape[1]) != self.feat_dim:
            raise ValueError(f"Feature dim mismatch between rendered feature ({self.feat_dim}) and text embedding "
                             f"({int(t.shape[1]) if t.ndim == 2 else tuple(t.shape)}).")
        tn = t / t.norm(dim=1, keepdim=True).clamp_min(1e-12)
        view = copy.copy(self)
        with torch.cuda.device(self.device):
            view.feat_attr = torch.matmul(self.feat_attr, tn.t()).contiguous()
        view.feat_dim = int(t.shape[0])
        view.feat16 = None          # the projected scores are not binary16 values
        view.c = view._struct()
        return view

    @property
    def has_f16(self) -> bool:
        return self.w16 is not None

    @property
    def has_bf16(self) -> bool:
        return self.wbf16 is not None

    def parameter_bytes(self) -> int:
        ts = [self.geom, self.W1, self.b1, self.W2, self.b2, self.W3, self.b3, self.w16, self.wbf16, self.feat_attr]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)


@dataclass
class FrameStats:
    pairs: int
    max_tile_len: int
    records: int        # MLP evaluations performed
    used: int           # records consumed by compositing
    waves: int
    wave_records: int
    work_items: int
    work_total: int = 0   # evaluator work items (blocks of at most 128 rows) of the whole frame
    pairs_kept: int = 0   # candidate pairs left after the tile pre-test (0 when it did not run)
    work_small: int = 0   # of work_total: small-group items (at most 32 rows)


class RenderError(RuntimeError):
    pass


def raise_for_status(bits: int, max_len: int, capacity: int, path_name: str):
    """Turn status bits into the reference's error messages."""
    if bits & L.BIT_BAD_OFFSETS:
        raise RenderError(f"{path_name}: tile_offsets must start at zero, end at the candidate-list length, "
                          "and be monotonic/in bounds")
    if bits & L.BIT_TILE_CAPACITY:
        raise RenderError(f"{path_name}: tile candidate capacity {capacity} exceeded (maximum observed tile "
                          f"length {max_len}); refusing to truncate or use an inconsistent forward/backward order")
    if bits & L.BIT_BAD_IDS:
        raise RenderError(f"{path_name}: candidate primitive IDs must be in [0, num_primitives)")
    if bits & L.BIT_TIMEOUT:
        raise RenderError(f"{path_name}: a device-side wait gave up (status bit {L.BIT_TIMEOUT}); frame discarded")


class FrameRenderer:
    """Owns the scratch and output buffers for frames of one shape on one GPU.

    max_records is the number of MLP evaluations one frame may perform (compositing slots are unique
    per frame); the scratch grows and the frame is rendered again when a frame needs more.
    """

    def __init__(self, width, height, device="cuda", tile_capacity=TILE_CAPACITY, max_pairs=None,
                 max_records=16_000_000, tile=TILE):
        """tile = 16 makes a renderer for the culling and ordering stages only (bin, sort): the wave kernels work on
        8x8 tiles, and render_tile16 of an 8x8 renderer hands such a renderer's lists down to them."""
        if int(tile) not in (8, 16):
            raise ValueError("tiles are 8x8 or 16x16")
        self.lib = L.load()
        self.device = torch.device(device)
        self.tile = int(tile)
        self.W, self.H = int(width), int(height)
        self.P = self.W * self.H
        self.T = ((self.W + self.tile - 1) // self.tile) * ((self.H + self.tile - 1) // self.tile)
        self.capacity = int(tile_capacity)
        self.max_pairs = int(max_pairs) if max_pairs is not None else min(self.T * self.capacity, 2**31 - 2)
        self.max_records = int(max_records)
        d = self.device
        self.tile_offsets = torch.zeros(self.T + 1, device=d, dtype=torch.int32)
        self.tile_prims = torch.empty(max(self.max_pairs, 1), device=d, dtype=torch.int32)
        self.sorted_prims = torch.empty(max(self.max_pairs, 1), device=d, dtype=torch.int32)
        self.rgb = torch.empty((self.P, 3), device=d, dtype=torch.float32)
        self.alpha = torch.empty((self.P, 1), device=d, dtype=torch.float32)
        self.depth_t = None
        self.mask_used = None
        self.feat = None
        self.rays_d_unit = torch.empty((self.P, 3), device=d, dtype=torch.float32)
        self.status = torch.zeros(L.STATUS_WORDS, device=d, dtype=torch.int32)
        self.status_host = torch.zeros(L.STATUS_WORDS, dtype=torch.int32).pin_memory()
        self.scratch = None
        self._scratch_key = None
        self._view = np.zeros(16, np.float32)
        self._proj = np.zeros(16, np.float32)
        self._bg = np.zeros(3, np.float32)
        self.last_stats: FrameStats | None = None
        self._last_frame = None
        self.f32_fallbacks = 0   # frames re-rendered in FP32 after an fp16 overflow

    # -- buffers ------------------------------------------------------------------------------
    def _ensure_scratch(self, n):
        key = (n, self.max_pairs, self.max_records)
        if self._scratch_key != key:
            nbytes = int(self.lib.mlpsp_frame_scratch_bytes(n, self.W, self.H, self.tile, self.max_pairs, self.max_records))
            if nbytes < 0:
                raise RuntimeError("mlpsp_frame_scratch_bytes rejected the frame shape")
            self.scratch = None
            self.scratch = torch.empty(nbytes + 256, device=self.device, dtype=torch.uint8)
            self._scratch_key = key
        return self.scratch

    def _frame(self, scene: PackedScene, rays_o, rays_d_unit, thr, precision, view, proj, bg, want_depth,
               want_mask_used, waves, want_feat=False, keep_records=False, sort_key=0, tile_rows=None,
               tile_pretest=True, prim_stats=None, tail_hint=False, hit_arith=0) -> L.Frame:
        f = L.Frame()
        f.rays_o, f.rays_d = L.ptr(rays_o), L.ptr(rays_d_unit)
        f.width, f.height, f.tile, f.threshold = self.W, self.H, self.tile, float(thr)
        f.tile_capacity, f.precision = self.capacity, int(precision)
        if view is not None:
            self._view[:] = np.asarray(view, dtype=np.float32).reshape(16)
            self._proj[:] = np.asarray(proj, dtype=np.float32).reshape(16)
            f.view, f.proj = self._view.ctypes.data, self._proj.ctypes.data
        f.tile_offsets, f.tile_prims, f.sorted_prims = L.ptr(self.tile_offsets), L.ptr(self.tile_prims), L.ptr(self.sorted_prims)
        f.max_pairs = self.max_pairs
        f.rgb, f.alpha = L.ptr(self.rgb), L.ptr(self.alpha)
        if want_depth:
            if self.depth_t is None:
                self.depth_t = torch.empty((self.P, 1), device=self.device, dtype=torch.float32)
            f.depth_t = L.ptr(self.depth_t)
        if want_feat:
            if scene.feat_attr is None:
                raise RuntimeError("feature rendering requested but the scene has no feat_attr")
            if self.feat is None or self.feat.shape[1] != scene.feat_dim:
                self.feat = torch.empty((self.P, scene.feat_dim), device=self.device, dtype=torch.float32)
            f.feat = L.ptr(self.feat)
        if want_mask_used:
            if self.mask_used is None:
                self.mask_used = torch.zeros(max(self.max_pairs, 1), device=self.device, dtype=torch.int64)
            f.mask_used = L.ptr(self.mask_used)
        if bg is not None:
            self._bg[:] = np.asarray(bg, dtype=np.float32).reshape(-1)[:3] if np.size(bg) >= 3 else float(np.asarray(bg).reshape(-1)[0])
            f.bg_color = self._bg.ctypes.data
        sc = self._ensure_scratch(scene.n)
        base = sc.data_ptr()
        aligned = (base + 255) // 256 * 256
        f.scratch, f.scratch_bytes = aligned, sc.numel() - (aligned - base)
        f.max_records = self.max_records
        f.keep_records = 1 if keep_records else 0
        f.sort_key = int(sort_key)
        f.tile_pretest = 0 if tile_pretest else 1
        f.tail_hint = 1 if tail_hint else 0
        f.hit_arith = int(hit_arith)
        if prim_stats is not None:
            gt, sum_w, max_w, hits, sum_werr, contrib = prim_stats
            f.gt_rgb, f.stat_sum_w, f.stat_max_w = L.ptr(gt), L.ptr(sum_w), L.ptr(max_w)
            f.stat_hits, f.stat_sum_werr, f.stat_contrib = L.ptr(hits), L.ptr(sum_werr), L.ptr(contrib)
        if tile_rows is not None:
            f.tile_row_begin, f.tile_row_end = int(tile_rows[0]), int(tile_rows[1])
        f.status = L.ptr(self.status)
        if waves:
            f.num_waves = len(waves)
            for i, w in enumerate(waves):
                f.wave_len[i] = int(w)
        return f

    def _read_status(self):
        self.status_host.copy_(self.status, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        s = self.status_host.numpy()
        u = s.view(np.uint32)
        rec = int(u[L.ST_RECORDS_LO]) | (int(u[L.ST_RECORDS_LO + 1]) << 32)
        used = int(u[L.ST_USED_LO]) | (int(u[L.ST_USED_LO + 1]) << 32)
        stats = FrameStats(int(s[L.ST_PAIRS]), int(s[L.ST_MAX_TILE_LEN]), rec, used, int(s[L.ST_WAVES]),
                           int(s[L.ST_WAVE_RECORDS]), int(s[L.ST_WORK_ITEMS]), int(s[L.ST_WORK_TOTAL]), int(s[L.ST_PAIRS_KEPT]),
                           int(s[L.ST_WORK_SMALL]))
        return int(s[L.ST_BITS]), stats

    def _grow(self, bits, stats):
        """Resize after an overflow finding; returns True when the frame should be retried."""
        if bits & L.BIT_PAIR_OVERFLOW:
            self.max_pairs = int(stats.pairs * 1.1) + 1024
            d = self.device
            self.tile_prims = torch.empty(self.max_pairs, device=d, dtype=torch.int32)
            self.sorted_prims = torch.empty(self.max_pairs, device=d, dtype=torch.int32)
            self.mask_used = None
            return True
        if bits & L.BIT_RECORD_OVERFLOW:
            self.max_records = int(max(stats.wave_records, self.max_records) * 2) + 4096
            return True
        return False

    # Wave schedule carried from frame to frame.  The library's default schedule ends in waves that most frames
    # never need; each of them still costs its launches.  After a frame whose status has been read, the next
    # frame is given the waves that one used plus a single catch-all wave, which keeps any frame correct (the
    # image does not depend on the schedule) and costs one idle wave instead of several.
    DEFAULT_WAVES = (32, 32, 64, 128, 256)

    def _adapt_waves(self, waves_used: int):
        n = int(waves_used)
        if n <= 0 or n > len(self.DEFAULT_WAVES):
            self._auto_waves = None
        else:
            self._auto_waves = list(self.DEFAULT_WAVES[:n]) + [self.capacity]

    # -- stages -------------------------------------------------------------------------------
    def render(self, scene: PackedScene, rays_o, rays_d, threshold, view=None, proj=None, precision=None,
               bg=None, want_depth=False, want_mask_used=False, waves=None, tile_lists=None,
               rays_normalized=False, check=True, path_name="render_tiles_forward_tilecenter", want_feat=False,
               keep_records=False, sort_key=0, tile_rows=None, tile_pretest=True, prim_stats=None, hit_arith=0,
               presorted=False):
        """One frame.  tile_lists=(culled_prim_indices, tile_offsets) replaces binning (external culling);
        presorted=True says those lists are already in compositing order (no per-tile sort).

        tile_pretest=False keeps every binned candidate in the lists the wave kernels walk (same image).
        prim_stats=(gt_rgb [P,3] f32, sum_w, max_w [n] f32, hits [n] i32, sum_werr [n] f32, contrib [n] i32): device
        tensors that receive the per-primitive contribution statistics of this frame (accumulated, not reset).
        hit_arith=1 computes the tile-centre key, the hit decision and the hit values in the reference kernels' own
        arithmetic (hardware exponential, compiler-contracted expressions) instead of the IEEE-only one: order, masks,
        record lists and CSR offsets are then those of the reference's kernels on the same GPU."""
        lib, d = self.lib, self.device
        if precision is None:
            precision = L.PRECISION_F16 if scene.has_f16 else L.PRECISION_F32
        auto = waves is None
        if auto:
            waves = getattr(self, "_auto_waves", None)
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            if rays_normalized:
                rd = rays_d
            else:
                L.check(lib.mlpsp_normalize_rows(L.ptr(rays_d), L.ptr(self.rays_d_unit), self.P, 3, st), "mlpsp_normalize_rows")
                rd = self.rays_d_unit
            for _attempt in range(8):
                L.check(lib.mlpsp_status_reset(L.ptr(self.status), st), "mlpsp_status_reset")
                if tile_lists is not None:
                    prims, offs = tile_lists
                    m = int(prims.numel())
                    if m > self.max_pairs:
                        self.max_pairs = m
                        self.tile_prims = torch.empty(max(m, 1), device=d, dtype=torch.int32)
                        self.sorted_prims = torch.empty(max(m, 1), device=d, dtype=torch.int32)
                        self.mask_used = None
                    self.tile_prims[:m].copy_(prims)
                    if presorted:
                        self.sorted_prims[:m].copy_(prims)
                    self.tile_offsets.copy_(offs)
                    L.check(lib.mlpsp_validate_tile_lists(L.ptr(self.tile_offsets), L.ptr(self.tile_prims), self.T, m,
                                                          self.capacity, scene.n, L.ptr(self.status), st),
                            "mlpsp_validate_tile_lists")
                f = self._frame(scene, rays_o, rd, threshold, precision, view, proj, bg, want_depth, want_mask_used, waves,
                                want_feat=want_feat, keep_records=keep_records, sort_key=sort_key, tile_rows=tile_rows,
                                tile_pretest=tile_pretest, prim_stats=prim_stats, tail_hint=auto and waves is not None,
                                hit_arith=hit_arith)
                self._last_frame = (f, scene)
                if tile_lists is None:
                    L.check(lib.mlpsp_render_frame(C.byref(scene.c), C.byref(f), st), "mlpsp_render_frame")
                else:
                    if not presorted:
                        L.check(lib.mlpsp_sort_tiles(C.byref(scene.c), C.byref(f), None, st), "mlpsp_sort_tiles")
                    L.check(lib.mlpsp_render_sorted(C.byref(scene.c), C.byref(f), st), "mlpsp_render_sorted")
                if not check:
                    return self.rgb, self.alpha
                bits, stats = self._read_status()
                self.last_stats = stats
                if auto and bits == 0 and sort_key != L.ORDER_PER_PIXEL:
                    self._adapt_waves(stats.waves)
                if bits & (L.BIT_BAD_OFFSETS | L.BIT_TILE_CAPACITY | L.BIT_BAD_IDS | L.BIT_TIMEOUT):
                    raise_for_status(bits, stats.max_tile_len, self.capacity, path_name)
                if self._grow(bits, stats):
                    continue
                if bits & L.BIT_PIXEL_HITS:
                    raise RenderError(f"{path_name}: per-pixel intersection capacity 256 exceeded; "
                                      "refusing to return a silently truncated result")
                if (bits & L.BIT_NUMERIC) and precision in (L.PRECISION_F16, L.PRECISION_BF16):
                    # operand/activation overflow in binary16: render the whole frame again in scalar
                    # FP32, as the reference does (rgb_wmma.cuh:260-272)
                    if scene.W1 is None:
                        raise RenderError(f"{path_name}: non-finite operand or activation in the fp16 evaluator and "
                                          "the scene holds no FP32 weights to render the frame again with")
                    self.f32_fallbacks += 1
                    precision = L.PRECISION_F32
                    continue
                return self.rgb, self.alpha
            raise RenderError(f"{path_name}: scratch kept overflowing after 8 attempts")

    def tile16_lists(self, scene: PackedScene, rays_o, rays_d_unit, threshold, view, proj, sort_key=0,
                     path_name="render_tiles_forward_tilecenter", lists16=None):
        """Culling and per-tile ordering on 16x16 tiles (the reference's tile_size = 16: np_tile_kernels.cu:483-518 keys
        on the centre ray of the 16x16 tile, candidate capacity per 16x16 tile), handed down to the 8x8 tiles the wave
        kernels work on: every 8x8 tile receives the ordered list of the 16x16 tile that contains it, so each pixel
        walks the same candidates in the same order as in the reference's 16x16 kernel.
        lists16 = (culled_prim_indices, tile_offsets) on the 16x16 grid replaces the culling (external lists).
        Returns (prims [M8] int32, tile_offsets [T8+1] int32) for render(..., tile_lists=..., presorted=True)."""
        if self.tile != 8:
            raise ValueError("tile16_lists belongs to the 8x8 renderer")
        d = self.device
        c = getattr(self, "_coarse", None)
        if c is None:
            c = self._coarse = FrameRenderer(self.W, self.H, device=d, tile_capacity=self.capacity, max_records=0, tile=16)
            ntx8, nty8 = (self.W + 7) // 8, (self.H + 7) // 8
            ntx16 = (self.W + 15) // 16
            ty8, tx8 = torch.meshgrid(torch.arange(nty8, device=d), torch.arange(ntx8, device=d), indexing="ij")
            self._parent16 = ((ty8 // 2) * ntx16 + tx8 // 2).reshape(-1)
        if lists16 is None:
            prims16, offs16 = c.bin(scene, view, proj, threshold, check=False)
            bits, stats = c._read_status()
        else:
            prims16, offs16 = lists16
            m = int(prims16.numel())
            if offs16.numel() != c.T + 1:
                raise ValueError(f"tile_offsets length mismatch: got {offs16.numel()}, expected {c.T + 1}")
            if m > c.max_pairs:
                c.max_pairs = m
                c.tile_prims = torch.empty(max(m, 1), device=d, dtype=torch.int32)
                c.sorted_prims = torch.empty(max(m, 1), device=d, dtype=torch.int32)
            c.tile_prims[:m].copy_(prims16)
            c.tile_offsets.copy_(offs16)
            with torch.cuda.device(d):
                st = _stream_ptr(d)
                L.check(self.lib.mlpsp_status_reset(L.ptr(c.status), st), "mlpsp_status_reset")
                L.check(self.lib.mlpsp_validate_tile_lists(L.ptr(c.tile_offsets), L.ptr(c.tile_prims), c.T, m, c.capacity,
                                                           scene.n, L.ptr(c.status), st), "mlpsp_validate_tile_lists")
            bits, stats = c._read_status()
            prims16, offs16 = c.tile_prims[:m], c.tile_offsets
        if bits & (L.BIT_TILE_CAPACITY | L.BIT_BAD_IDS | L.BIT_BAD_OFFSETS):
            raise_for_status(bits, stats.max_tile_len, self.capacity, path_name)
        pairs16 = int(prims16.numel())
        sorted16 = c.sort(scene, rays_o, rays_d_unit, pairs16, sort_key=sort_key)
        offs16 = offs16.to(torch.int64)
        len8 = (offs16[1:] - offs16[:-1])[self._parent16]
        offs8 = torch.zeros(self.T + 1, device=d, dtype=torch.int64)
        torch.cumsum(len8, 0, out=offs8[1:])
        total8 = int(offs8[-1])
        if total8 >= 2**31:
            raise RenderError(f"{path_name}: candidate list is too large for int32 offsets")
        tile8 = torch.repeat_interleave(torch.arange(self.T, device=d), len8, output_size=total8)
        src = offs16[self._parent16[tile8]] + (torch.arange(total8, device=d) - offs8[tile8])
        return sorted16[src].contiguous(), offs8.to(torch.int32)

    def render_tile16(self, scene: PackedScene, rays_o, rays_d, threshold, view=None, proj=None, rays_normalized=False,
                      sort_key=0, path_name="render_tiles_forward_tilecenter", tile_lists=None, **kw):
        """One frame with the reference's tile_size = 16 semantics (see tile16_lists); other arguments as render(),
        tile_lists on the 16x16 grid."""
        with torch.cuda.device(self.device):
            rd = rays_d if rays_normalized else normalize_rows(rays_d)
            prims8, offs8 = self.tile16_lists(scene, rays_o, rd, threshold, view, proj, sort_key=sort_key, path_name=path_name,
                                              lists16=tile_lists)
            return self.render(scene, rays_o, rd, threshold, tile_lists=(prims8, offs8), presorted=True, rays_normalized=True,
                               sort_key=sort_key, path_name=path_name, **kw)

    def render_records(self, scene: PackedScene, rays_o, rays_d, threshold, max_hits=512, **kw):
        """Render and return the reference's record list [rgb, alpha, ids, x6, raw, masks, gates, offsets]
        (render_tiles_training_records, np_tile_kernels.cu:6897-6986): pixel-major, compositing order."""
        lib, d = self.lib, self.device
        rgb, alpha = self.render(scene, rays_o, rays_d, threshold, keep_records=True, **kw)
        f, _ = self._last_frame
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            offsets = torch.empty(self.P + 1, device=d, dtype=torch.int64)
            total, worst = C.c_int64(0), C.c_int32(0)
            L.check(lib.mlpsp_export_records(C.byref(scene.c), C.byref(f), L.ptr(offsets), None, None, None, None, None, 0,
                                             int(max_hits), C.byref(total), C.byref(worst), st), "mlpsp_export_records")
            if worst.value < 0:
                raise RenderError(f"render_tiles_training_records: tile-center backward hit capacity {max_hits} reached "
                                  "before transmittance termination; refusing to return truncated records")
            R = int(total.value)
            ids = torch.empty(R, device=d, dtype=torch.int32)
            x6 = torch.empty((R, 6), device=d, dtype=torch.float32)
            raw = torch.empty((R, 8), device=d, dtype=torch.float32)
            masks = torch.empty((R, 2), device=d, dtype=torch.int32)
            gates = torch.empty((R, 4), device=d, dtype=torch.float32)
            if R > 0:
                L.check(lib.mlpsp_export_records(C.byref(scene.c), C.byref(f), L.ptr(offsets), L.ptr(ids), L.ptr(x6),
                                                 L.ptr(raw), L.ptr(masks), L.ptr(gates), R, int(max_hits),
                                                 C.byref(total), C.byref(worst), st), "mlpsp_export_records")
        return [rgb.clone(), alpha.clone(), ids, x6, raw, masks, gates, offsets]

    def bin(self, scene: PackedScene, view, proj, threshold, check=True):
        """Binning only: returns (culled_prim_indices[M] int32, tile_offsets[T+1] int32) views."""
        lib, d = self.lib, self.device
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            for _attempt in range(3):
                L.check(lib.mlpsp_status_reset(L.ptr(self.status), st), "mlpsp_status_reset")
                f = self._frame(scene, None, None, threshold, 0, view, proj, None, False, False, None)
                L.check(lib.mlpsp_bin_tiles(C.byref(scene.c), C.byref(f), st), "mlpsp_bin_tiles")
                bits, stats = self._read_status()
                self.last_stats = stats
                if check and (bits & L.BIT_TILE_CAPACITY):
                    raise_for_status(bits, stats.max_tile_len, self.capacity, "mlpsp_bin_tiles")
                if bits & L.BIT_PAIR_OVERFLOW and self._grow(bits, stats):
                    continue
                return self.tile_prims[:stats.pairs], self.tile_offsets
            raise RenderError("mlpsp_bin_tiles: pair buffer kept overflowing")

    def bin_mosaic(self, scene: PackedScene, tile_view_ids, view_matrices, proj, threshold):
        """Culling for a mosaic frame: tile t is seen from view tile_view_ids[t] (cumodel.py:838-949)."""
        lib, d = self.lib, self.device
        tv = torch.as_tensor(tile_view_ids).to(device=d, dtype=torch.int32).reshape(-1).contiguous()
        if tv.numel() != self.T:
            raise ValueError(f"tile_view_ids length mismatch: got {tv.numel()}, expected {self.T}")
        views = np.ascontiguousarray(np.asarray(view_matrices, dtype=np.float32).reshape(-1, 16))
        if views.shape[0] <= 0:
            raise ValueError("view_matrices must contain at least one view")
        if int(tv.min()) < 0 or int(tv.max()) >= views.shape[0]:
            raise ValueError("tile_view_ids contains out-of-range view indices")
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            for _attempt in range(3):
                L.check(lib.mlpsp_status_reset(L.ptr(self.status), st), "mlpsp_status_reset")
                f = self._frame(scene, None, None, threshold, 0, views[0], proj, None, False, False, None)
                L.check(lib.mlpsp_bin_tiles_mosaic(C.byref(scene.c), C.byref(f), L.ptr(tv), views.ctypes.data,
                                                   views.shape[0], st), "mlpsp_bin_tiles_mosaic")
                bits, stats = self._read_status()
                self.last_stats = stats
                if bits & L.BIT_TILE_CAPACITY:
                    raise_for_status(bits, stats.max_tile_len, self.capacity, "mlpsp_bin_tiles_mosaic")
                if bits & L.BIT_PAIR_OVERFLOW and self._grow(bits, stats):
                    continue
                return self.tile_prims[:stats.pairs], self.tile_offsets
            raise RenderError("mlpsp_bin_tiles_mosaic: pair buffer kept overflowing")

    def bin_raycone(self, scene: PackedScene, rays_o, rays_d, threshold):
        """Ray-cone culling from the actual rays (scannet/camera.py:102-146): (ids, offsets, status bits)."""
        lib, d = self.lib, self.device
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            for _attempt in range(3):
                L.check(lib.mlpsp_status_reset(L.ptr(self.status), st), "mlpsp_status_reset")
                f = self._frame(scene, rays_o, rays_d, threshold, 0, None, None, None, False, False, None)
                L.check(lib.mlpsp_bin_tiles_raycone(C.byref(scene.c), C.byref(f), st), "mlpsp_bin_tiles_raycone")
                bits, stats = self._read_status()
                self.last_stats = stats
                if bits & (L.BIT_TILE_ORIGINS | L.BIT_CONE_TOO_WIDE):
                    return self.tile_prims[:0], self.tile_offsets, bits
                if bits & L.BIT_TILE_CAPACITY:
                    raise_for_status(bits, stats.max_tile_len, self.capacity, "mlpsp_bin_tiles_raycone")
                if bits & L.BIT_PAIR_OVERFLOW and self._grow(bits, stats):
                    continue
                return self.tile_prims[:stats.pairs], self.tile_offsets, bits
            raise RenderError("mlpsp_bin_tiles_raycone: pair buffer kept overflowing")

    def sort(self, scene: PackedScene, rays_o, rays_d_unit, pairs, want_keys=False, sort_key=0, hit_arith=0):
        lib, d = self.lib, self.device
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            f = self._frame(scene, rays_o, rays_d_unit, 0.5, 0, None, None, None, False, False, None, sort_key=sort_key,
                            hit_arith=hit_arith)
            keys = torch.empty(max(pairs, 1), device=d, dtype=torch.float32) if want_keys else None
            L.check(lib.mlpsp_sort_tiles(C.byref(scene.c), C.byref(f), L.ptr(keys), st), "mlpsp_sort_tiles")
            return (self.sorted_prims[:pairs], keys[:pairs]) if want_keys else self.sorted_prims[:pairs]

    def hit_masks(self, scene: PackedScene, rays_o, rays_d_unit, threshold, pairs, hit_arith=0):
        lib, d = self.lib, self.device
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            f = self._frame(scene, rays_o, rays_d_unit, threshold, 0, None, None, None, False, False, None, hit_arith=hit_arith)
            out = torch.zeros(max(pairs, 1), device=d, dtype=torch.int64)
            L.check(lib.mlpsp_hit_masks(C.byref(scene.c), C.byref(f), L.ptr(out), st), "mlpsp_hit_masks")
            return out[:pairs]


class ViewBatchRenderer:
    """Several views of one scene per call (mlpsp_render_frames): one evaluator launch per wave serves all views.

    The reference renders view by view.  In a scene with many primitives a primitive owns only a few records per
    view, and the evaluator then spends its time streaming weight images (9.5 or 22.8 KB per primitive, wave and
    view); rendering a batch of views together lets a primitive's records of all views share one fetch.  Every
    view keeps its own tile lists, masks, pixel state and outputs (a FrameRenderer each); the per-primitive arrays
    and the record arrays are the first view's, sized for the whole batch.  rgb and alpha only; images are
    bit-identical to FrameRenderer.render.
    """

    def __init__(self, width, height, num_views, device="cuda", tile_capacity=TILE_CAPACITY, max_pairs=None,
                 max_records=16_000_000):
        if not 1 <= int(num_views) <= 64:
            raise ValueError("num_views must be in [1, 64]")
        self.V = int(num_views)
        self.device = torch.device(device)
        # the first renderer's scratch carries the record arrays of the batch; the others need none
        self.views = [FrameRenderer(width, height, device=device, tile_capacity=tile_capacity, max_pairs=max_pairs,
                                    max_records=(int(max_records) if v == 0 else 0)) for v in range(self.V)]
        self.lead = self.views[0]
        self.lib = self.lead.lib
        self.last_stats: FrameStats | None = None
        self.f32_fallbacks = 0
        self._auto_waves = None

    def render(self, scene: PackedScene, rays_o, rays_d, threshold, views, projs, precision=None, bg=None, waves=None,
               rays_normalized=False, path_name="render_tiles_forward_tilecenter", hit_arith=0):
        """rays_o / rays_d / views / projs: one entry per view.  Returns [(rgb [P,3], alpha [P,1])] per view (the
        renderers' own buffers, valid until the next call)."""
        if not (len(rays_o) == len(rays_d) == len(views) == len(projs) == self.V):
            raise ValueError(f"expected {self.V} views")
        lib, d, lead = self.lib, self.device, self.lead
        if precision is None:
            precision = L.PRECISION_F16 if scene.has_f16 else L.PRECISION_F32
        auto = waves is None
        if auto:
            waves = self._auto_waves
        with torch.cuda.device(d):
            st = _stream_ptr(d)
            rds = []
            for v, r in enumerate(self.views):
                if rays_normalized:
                    rds.append(rays_d[v])
                else:
                    L.check(lib.mlpsp_normalize_rows(L.ptr(rays_d[v]), L.ptr(r.rays_d_unit), r.P, 3, st), "mlpsp_normalize_rows")
                    rds.append(r.rays_d_unit)
            for _attempt in range(10):
                L.check(lib.mlpsp_status_reset(L.ptr(lead.status), st), "mlpsp_status_reset")
                frames = (L.Frame * self.V)()
                for v, r in enumerate(self.views):
                    f = r._frame(scene, rays_o[v], rds[v], threshold, precision, views[v], projs[v], bg, False, False, waves,
                                 tail_hint=auto and waves is not None, hit_arith=hit_arith)
                    f.status = L.ptr(lead.status)
                    frames[v] = f
                L.check(lib.mlpsp_render_frames(C.byref(scene.c), frames, self.V, st), "mlpsp_render_frames")
                bits, stats = lead._read_status()
                self.last_stats = stats
                if auto and bits == 0:
                    n = int(stats.waves)
                    self._auto_waves = (list(FrameRenderer.DEFAULT_WAVES[:n]) + [lead.capacity]
                                        if 0 < n <= len(FrameRenderer.DEFAULT_WAVES) else None)
                if bits & (L.BIT_BAD_OFFSETS | L.BIT_TILE_CAPACITY | L.BIT_BAD_IDS | L.BIT_TIMEOUT):
                    raise_for_status(bits, stats.max_tile_len, lead.capacity, path_name)
                if bits & L.BIT_PAIR_OVERFLOW:
                    # the status block is shared, so which view ran out is not known: all lists grow
                    grown = max(int(lead.max_pairs * 1.5) + 1024, int(stats.pairs * 1.1) + 1024)
                    for r in self.views:
                        r.max_pairs = min(grown, r.T * r.capacity)
                        r.tile_prims = torch.empty(r.max_pairs, device=d, dtype=torch.int32)
                        r.sorted_prims = torch.empty(r.max_pairs, device=d, dtype=torch.int32)
                    continue
                if bits & L.BIT_RECORD_OVERFLOW:
                    lead.max_records = int(max(stats.wave_records, lead.max_records) * 2) + 4096
                    continue
                if (bits & L.BIT_NUMERIC) and precision in (L.PRECISION_F16, L.PRECISION_BF16):
                    if scene.W1 is None:
                        raise RenderError(f"{path_name}: non-finite operand or activation in the fp16 evaluator and "
                                          "the scene holds no FP32 weights to render the frames again with")
                    self.f32_fallbacks += 1
                    precision = L.PRECISION_F32
                    continue
                return [(r.rgb, r.alpha) for r in self.views]
            raise RenderError(f"{path_name}: scratch kept overflowing after 10 attempts")


class FramePipeline:
    """Several frames in flight on one GPU: per slot a stream, a FrameRenderer and device ray buffers.

    submit() enqueues host->device ray copies, the frame and the device->host image copy on the
    slot's stream and returns at once; wait() synchronises that stream and raises on a bad status.
    Host arrays should be pinned so the copies overlap the previous frames' kernels.
    """

    def __init__(self, scene: PackedScene, width, height, depth=3, **renderer_kw):
        self.scene = scene
        d = scene.device
        self.slots = []
        for _ in range(int(depth)):
            r = FrameRenderer(width, height, device=d, **renderer_kw)
            self.slots.append(dict(r=r, stream=torch.cuda.Stream(device=d), busy=False,
                                   ro=torch.empty((r.P, 3), device=d), rd=torch.empty((r.P, 3), device=d),
                                   ro1=torch.empty((1, 3), device=d), kw=None))
        self.next_slot = 0

    def submit(self, rays_o_host, rays_d_host, threshold, view, proj, out_rgb_host=None, out_alpha_host=None,
               precision=None, bg=None, tile_rows=None):
        i = self.next_slot
        s = self.slots[i]
        if s["busy"]:
            self.wait(i)
        self.next_slot = (i + 1) % len(self.slots)
        r = s["r"]
        with torch.cuda.stream(s["stream"]):
            if rays_o_host.shape[0] == 1 and r.P != 1:
                # one origin for every ray (a pinhole camera): 12 bytes cross the bus, the rows are written on the device
                s["ro1"].copy_(rays_o_host, non_blocking=True)
                s["ro"].copy_(s["ro1"].expand(r.P, 3))
            else:
                s["ro"].copy_(rays_o_host, non_blocking=True)
            s["rd"].copy_(rays_d_host, non_blocking=True)
            kw = dict(view=view, proj=proj, precision=precision, bg=bg, tile_rows=tile_rows)
            rgb, alpha = r.render(self.scene, s["ro"], s["rd"], threshold, check=False, **kw)
            self._to_host(rgb, out_rgb_host)
            self._to_host(alpha, out_alpha_host)
            r.status_host.copy_(r.status, non_blocking=True)
        s["busy"], s["kw"] = True, (threshold, kw, out_rgb_host, out_alpha_host)
        return i

    @staticmethod
    def _to_host(src, dst):
        """Device image -> (pinned) host tensor; a host tensor of another dtype (float16, say) is converted to on the
        device first, so only its bytes cross the bus."""
        if dst is None:
            return
        dst.copy_(src if dst.dtype == src.dtype else src.to(dst.dtype), non_blocking=True)

    def wait(self, i):
        s = self.slots[i]
        if not s["busy"]:
            return
        r = s["r"]
        s["stream"].synchronize()
        s["busy"] = False
        bits = int(r.status_host[L.ST_BITS])
        if bits == 0:
            r._adapt_waves(int(r.status_host[L.ST_WAVES]))
            return
        # rare path: overflow / error / fp16 overflow -> redo this frame synchronously with full checks
        threshold, kw, out_rgb, out_alpha = s["kw"]
        with torch.cuda.stream(s["stream"]):
            rgb, alpha = r.render(self.scene, s["ro"], s["rd"], threshold, check=True, **kw)
            self._to_host(rgb, out_rgb)
            self._to_host(alpha, out_alpha)
        s["stream"].synchronize()

    def drain(self):
        for i in range(len(self.slots)):
            self.wait(i)
