"""ctypes/numpy front end of the CPU oracle (oracle/mlpsp_oracle.c).

TEST INFRASTRUCTURE ONLY.  The product package never imports this module; the tests, the
smoke check and the benchmark's CPU-baseline leg are the only callers.

The functions mirror the stages of the reference renderer (scannet/cumodel.py forward and
scannet/cuda/np_tile_kernels.cu render_tiles_kernel_tilecenter_order) and the record helpers
(scannet/primitive_csr.py:23-29, scannet/primitive_gemm.py:186-203); each C function cites the
lines it follows.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import build as _build

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        here = os.path.dirname(os.path.abspath(__file__))
        path = os.path.join(here, "liboracle.so")
        if not os.path.exists(path) or (os.path.exists(_build.SRC) and
                                        os.path.getmtime(path) < os.path.getmtime(_build.SRC)):
            path = _build.build(force=True)
        _LIB = C.CDLL(path)
        _LIB.orc_det_exp.restype = C.c_float
        _LIB.orc_det_exp.argtypes = [C.c_float]
        _LIB.orc_f16_round.restype = C.c_float
        _LIB.orc_f16_round.argtypes = [C.c_float]
        _LIB.orc_radius_multiplier.restype = C.c_float
        _LIB.orc_radius_multiplier.argtypes = [C.c_float]
        _LIB.orc_bin_count.restype = C.c_int64
        _LIB.orc_bin_mosaic.restype = C.c_int64
        assert _LIB.orc_sizeof_render() == C.sizeof(_Render), "render_t layout mismatch"
    return _LIB


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a, ty=C.c_float):
    return None if a is None else a.ctypes.data_as(C.POINTER(ty))


class _Mlp(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in ("W1", "b1", "W2", "b2", "W3", "b3", "freq", "att")] + \
               [("F", C.c_int), ("H", C.c_int), ("IN", C.c_int), ("precision", C.c_int)]


class _Render(C.Structure):
    _fields_ = [
        ("rays_o", C.POINTER(C.c_float)), ("rays_d", C.POINTER(C.c_float)),
        ("geom", C.POINTER(C.c_float)), ("n", C.c_int),
        ("tile_offsets", C.POINTER(C.c_int32)), ("sorted_prims", C.POINTER(C.c_int32)),
        ("W", C.c_int), ("H", C.c_int), ("ts", C.c_int), ("thr", C.c_float),
        ("mlp", _Mlp),
        ("feat_attr", C.POINTER(C.c_float)), ("feat_slots", C.c_int), ("feat_dim", C.c_int),
        ("beta", C.c_float), ("tau", C.c_float),
        ("tile_begin", C.c_int), ("tile_end", C.c_int),
        ("rgb", C.POINTER(C.c_float)), ("alpha", C.POINTER(C.c_float)),
        ("depth_t", C.POINTER(C.c_float)), ("feat", C.POINTER(C.c_float)),
        ("mask_geo", C.POINTER(C.c_uint64)), ("mask_used", C.POINTER(C.c_uint64)),
        ("min_margin", C.POINTER(C.c_float)), ("rec_count", C.POINTER(C.c_int32)),
        ("rec_offsets", C.POINTER(C.c_int64)),
        ("rec_ids", C.POINTER(C.c_int32)), ("rec_x6", C.POINTER(C.c_float)),
        ("rec_raw", C.POINTER(C.c_float)), ("rec_masks", C.POINTER(C.c_int32)),
        ("rec_gates", C.POINTER(C.c_float)),
        ("gt_rgb", C.POINTER(C.c_float)), ("stat_sum_w", C.POINTER(C.c_float)), ("stat_max_w", C.POINTER(C.c_float)),
        ("stat_hits", C.POINTER(C.c_int32)), ("stat_sum_werr", C.POINTER(C.c_float)), ("stat_contrib", C.POINTER(C.c_int32)),
        ("evals", C.c_int64),
    ]


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> int:
    """Use n OpenMP threads from here on (launchers such as torch.distributed.run export OMP_NUM_THREADS=1)."""
    lib().orc_set_num_threads(int(n))
    return num_threads()


def host_cores() -> int:
    """Cores this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def det_exp(x):
    f = lib().orc_det_exp
    return np.array([f(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()], dtype=np.float32)


def f16_round(x):
    f = lib().orc_f16_round
    a = np.asarray(x, dtype=np.float32)
    return np.array([f(float(v)) for v in a.ravel()], dtype=np.float32).reshape(a.shape)


def normalize_rows(a):
    a = _f32(a)
    out = np.empty_like(a)
    lib().orc_normalize_rows(_p(a), _p(out), C.c_int64(a.shape[0]), C.c_int(a.shape[1]))
    return out


def pack_geometry(positions, log_scales, quats_unit):
    pos, ls, q = _f32(positions), _f32(log_scales), _f32(quats_unit)
    n = pos.shape[0]
    geom = np.empty((n, 16), np.float32)
    lib().orc_pack_geometry(_p(pos), _p(ls), _p(q), C.c_int(n), _p(geom))
    return geom


def bin_tiles(geom, view, proj, W, H, tile, thr):
    """Screen-space culling (cumodel.py:994-1070): returns (culled_prim_indices, tile_offsets)."""
    geom, view, proj = _f32(geom), _f32(view).reshape(16), _f32(proj).reshape(16)
    T = ((W + tile - 1) // tile) * ((H + tile - 1) // tile)
    off = np.zeros(T + 1, np.int32)
    n = geom.shape[0]
    total = lib().orc_bin_count(_p(geom), C.c_int(n), _p(view), _p(proj), C.c_int(W), C.c_int(H),
                                C.c_int(tile), C.c_float(thr), _p(off, C.c_int32))
    prims = np.empty(int(total), np.int32)
    lib().orc_bin_fill(_p(geom), C.c_int(n), _p(view), _p(proj), C.c_int(W), C.c_int(H),
                       C.c_int(tile), C.c_float(thr), _p(off, C.c_int32), _p(prims, C.c_int32))
    return prims, off


def bin_tiles_mosaic(geom, views, tile_view_ids, proj, W, H, tile, thr):
    """Per-tile-view culling (cumodel.py:838-949): returns (culled_prim_indices, tile_offsets)."""
    geom, views, proj = _f32(geom), _f32(views).reshape(-1, 16), _f32(proj).reshape(16)
    tv = _i32(tile_view_ids)
    off = np.zeros(tv.size + 1, np.int32)
    args = (_p(geom), C.c_int(geom.shape[0]), _p(views), C.c_int(views.shape[0]), _p(tv, C.c_int32), _p(proj),
            C.c_int(W), C.c_int(H), C.c_int(tile), C.c_float(thr), _p(off, C.c_int32))
    total = lib().orc_bin_mosaic(*args, None)
    prims = np.empty(int(total), np.int32)
    lib().orc_bin_mosaic(*args, _p(prims, C.c_int32))
    return prims, off


def ray_cone_candidates(rays_o, rays_d, geom, W, H, thr):
    """Ray-cone culling (scannet/camera.py:102-146): returns (ids, offsets, status bits)."""
    ro, rd, geom = _f32(rays_o), _f32(rays_d), _f32(geom)
    T = ((W + 7) // 8) * ((H + 7) // 8)
    off = np.zeros(T + 1, np.int32)
    total = C.c_int64(0)
    args = (_p(geom), C.c_int(geom.shape[0]), _p(ro), _p(rd), C.c_int(W), C.c_int(H), C.c_float(thr), _p(off, C.c_int32))
    st = lib().orc_bin_raycone(*args, None, C.byref(total))
    prims = np.empty(int(total.value), np.int32)
    if st == 0:
        lib().orc_bin_raycone(*args, _p(prims, C.c_int32), C.byref(total))
    return prims, off, int(st)


def validate_lists(tile_offsets, prims, capacity, n):
    off, pr = _i32(tile_offsets), _i32(prims)
    st = np.zeros(2, np.int32)
    lib().orc_validate_lists(_p(off, C.c_int32), _p(pr, C.c_int32), C.c_int(off.size - 1), C.c_int(pr.size),
                             C.c_int(capacity), C.c_int(n), _p(st, C.c_int32))
    return int(st[0]), int(st[1])


def sort_tiles(rays_o, rays_d, geom, tile_offsets, tile_prims, W, H, tile, want_keys=False, key_mode=0):
    ro, rd, geom = _f32(rays_o), _f32(rays_d), _f32(geom)
    off, pr = _i32(tile_offsets), _i32(tile_prims)
    out = np.empty_like(pr)
    keys = np.empty(pr.size, np.float32) if want_keys else None
    lib().orc_sort_tiles(_p(ro), _p(rd), _p(geom), C.c_int(geom.shape[0]), _p(off, C.c_int32),
                         _p(pr, C.c_int32), C.c_int(W), C.c_int(H), C.c_int(tile), _p(out, C.c_int32), _p(keys),
                         C.c_int(key_mode))
    return (out, keys) if want_keys else out


def mlp_eval(weights, freq, att, prim_ids, x6, precision=0):
    """(R,G,B,sigma_raw) per record: cumodel.py:183-216 / np_tile_kernels.cu:312-380."""
    W1, b1, W2, b2, W3, b3 = [_f32(w) for w in weights]
    freq, att, x6, ids = _f32(freq), _f32(att), _f32(x6), _i32(prim_ids)
    out = np.empty((ids.size, 4), np.float32)
    lib().orc_mlp_eval(_p(W1), _p(b1), _p(W2), _p(b2), _p(W3), _p(b3), _p(freq), _p(att),
                       C.c_int(freq.size), C.c_int(W1.shape[1]), C.c_int(precision),
                       _p(ids, C.c_int32), _p(x6), C.c_int64(ids.size), _p(out))
    return out


@dataclass
class RenderResult:
    rgb: np.ndarray
    alpha: np.ndarray
    depth_t: np.ndarray
    feat: np.ndarray | None
    mask_geo: np.ndarray | None
    mask_used: np.ndarray | None
    min_margin: np.ndarray
    rec_count: np.ndarray
    evals: int
    records: dict | None = None
    stats: dict | None = None


def render(rays_o, rays_d_unit, geom, tile_offsets, sorted_prims, W, H, tile, thr, weights, freq, att,
           precision=0, feat_attr=None, beta=1.5, tau=2.0, want_masks=True, want_records=False,
           tile_range=None, gt_rgb=None) -> RenderResult:
    """Tile-major front-to-back render of depth-sorted tile lists (np_tile_kernels.cu:1837-2137)."""
    ro, rd, geom = _f32(rays_o), _f32(rays_d_unit), _f32(geom)
    off, sp = _i32(tile_offsets), _i32(sorted_prims)
    W1, b1, W2, b2, W3, b3 = [_f32(w) for w in weights]
    freq, att = _f32(freq), _f32(att)
    P = W * H
    T = off.size - 1
    a = _Render()
    keep = [ro, rd, geom, off, sp, W1, b1, W2, b2, W3, b3, freq, att]
    a.rays_o, a.rays_d, a.geom, a.n = _p(ro), _p(rd), _p(geom), geom.shape[0]
    a.tile_offsets, a.sorted_prims = _p(off, C.c_int32), _p(sp, C.c_int32)
    a.W, a.H, a.ts, a.thr = W, H, tile, thr
    a.mlp = _Mlp(_p(W1), _p(b1), _p(W2), _p(b2), _p(W3), _p(b3), _p(freq), _p(att),
                 freq.size, W1.shape[1], 12 * freq.size, precision)
    feat = None
    if feat_attr is not None:
        fa = _f32(feat_attr)
        if fa.ndim == 2:
            fa = fa[:, None, :]
        keep.append(fa)
        feat = np.zeros((P, fa.shape[2]), np.float32)
        a.feat_attr, a.feat_slots, a.feat_dim, a.feat = _p(fa), fa.shape[1], fa.shape[2], _p(feat)
    a.beta, a.tau = beta, tau
    a.tile_begin, a.tile_end = (0, T) if tile_range is None else tile_range
    rgb = np.zeros((P, 3), np.float32)
    alpha = np.zeros(P, np.float32)
    dt = np.zeros(P, np.float32)
    marg = np.full(P, 1e30, np.float32)
    cnt = np.zeros(P, np.int32)
    a.rgb, a.alpha, a.depth_t, a.min_margin, a.rec_count = _p(rgb), _p(alpha), _p(dt), _p(marg), _p(cnt, C.c_int32)
    mg = mu = None
    if want_masks and tile == 8:
        mg = np.zeros(sp.size, np.uint64)
        mu = np.zeros(sp.size, np.uint64)
        a.mask_geo, a.mask_used = _p(mg, C.c_uint64), _p(mu, C.c_uint64)
    stats = None
    if gt_rgb is not None:
        # per-primitive contribution statistics (np_tile_kernels.cu:2143-2500), starting from zero
        gt = _f32(gt_rgb).reshape(P, 3)
        keep.append(gt)
        n = geom.shape[0]
        stats = dict(sum_w=np.zeros(n, np.float32), max_w=np.zeros(n, np.float32), hits=np.zeros(n, np.int32),
                     sum_werr=np.zeros(n, np.float32), contrib=np.zeros(n, np.int32))
        a.gt_rgb = _p(gt)
        a.stat_sum_w, a.stat_max_w, a.stat_hits = _p(stats["sum_w"]), _p(stats["max_w"]), _p(stats["hits"], C.c_int32)
        a.stat_sum_werr, a.stat_contrib = _p(stats["sum_werr"]), _p(stats["contrib"], C.c_int32)
    lib().orc_render(C.byref(a))
    res = RenderResult(rgb, alpha, dt, feat, mg, mu, marg, cnt, int(a.evals))
    res.stats = stats
    if want_records:
        offs = np.zeros(P + 1, np.int64)
        np.cumsum(cnt, out=offs[1:])
        R = int(offs[-1])
        rec = dict(offsets=offs, ids=np.empty(R, np.int32), x6=np.empty((R, 6), np.float32),
                   raw=np.empty((R, 8), np.float32), masks=np.empty((R, 2), np.int32),
                   gates=np.empty((R, 4), np.float32))
        a.rec_offsets = _p(offs, C.c_int64)
        a.rec_ids, a.rec_x6, a.rec_raw = _p(rec["ids"], C.c_int32), _p(rec["x6"]), _p(rec["raw"])
        a.rec_masks, a.rec_gates = _p(rec["masks"], C.c_int32), _p(rec["gates"])
        if feat is not None:
            feat[:] = 0
        lib().orc_render(C.byref(a))
        res.records = rec
    del keep
    return res


# ---- record grouping: scannet/primitive_csr.py:23-29 and scannet/primitive_gemm.py:186-203 ----

def group_records(primitive_ids, num_primitives):
    """Stable grouping by primitive: (offsets int64 [N+1], order int64 [R])."""
    ids = np.asarray(primitive_ids).astype(np.int64)
    order = np.argsort(ids, kind="stable")
    counts = np.bincount(ids, minlength=num_primitives)
    offsets = np.concatenate(([0], np.cumsum(counts))).astype(np.int64)
    return offsets, order.astype(np.int64)


def prepare_groups(offsets, segment_size=512):
    """Segments of at most segment_size records: (primitives [G], starts [G], group_offsets [N+1])."""
    offsets = np.asarray(offsets, dtype=np.int64)
    counts = -(-np.diff(offsets) // segment_size)
    group_offsets = np.concatenate(([0], np.cumsum(counts))).astype(np.int64)
    primitives = np.repeat(np.arange(counts.size, dtype=np.int64), counts)
    local = np.arange(primitives.size, dtype=np.int64) - group_offsets[primitives]
    starts = offsets[primitives] + local * segment_size
    return primitives, starts, group_offsets


def decode_features(x_hwc, weights, precision=0):
    """FeatureUpsampleDecoder on a pixel-major map x [H, W, Cin] (scannet/feature_decoder.py:5-19).
    weights: dict with net.0/2/4 .weight/.bias in torch Conv2d layout (numpy).  Returns [H, W, Cout] float32.
    precision 1 / 2: binary16 / bfloat16 operands and hidden activations, FP32 accumulation."""
    x = _f32(x_hwc)
    H, W, Cin = x.shape
    W1, b1 = _f32(weights["net.0.weight"]).reshape(-1, Cin), _f32(weights["net.0.bias"])
    Ch = W1.shape[0]
    W2, b2 = _f32(weights["net.2.weight"]).reshape(Ch, Ch, 3, 3), _f32(weights["net.2.bias"])
    W3, b3 = _f32(weights["net.4.weight"]).reshape(-1, Ch), _f32(weights["net.4.bias"])
    Cout = W3.shape[0]
    out = np.empty((H, W, Cout), np.float32)
    lib().orc_decode_features(_p(x), C.c_int(W), C.c_int(H), C.c_int(Cin), C.c_int(Ch), C.c_int(Cout),
                              _p(W1), _p(b1), _p(W2), _p(b2), _p(W3), _p(b3), C.c_int(precision), _p(out))
    return out


def classify_features(feat, text):
    """_classify_feature_map (scannet/eval_lseg_table2.py:622-641) on feat [..., D] and text [C, D].
    Returns (labels int64 [...], margin float32 [...] = best cosine logit - second best)."""
    f = _f32(feat)
    t = _f32(text)
    D = f.shape[-1]
    P = f.size // D
    labels = np.empty(P, np.int64)
    margin = np.empty(P, np.float32)
    lib().orc_classify_features(_p(f), C.c_int64(P), C.c_int(D), _p(t), C.c_int(t.shape[0]),
                                labels.ctypes.data_as(C.POINTER(C.c_int64)), _p(margin))
    return labels.reshape(f.shape[:-1]), margin.reshape(f.shape[:-1])


def render_per_pixel(rays_o, rays_d_unit, geom, tile_offsets, prims, W, H, tile, thr, weights, freq, att, precision=0,
                     feat_attr=None, beta=1.5, tau=2.0):
    """Per-pixel exact ordering (render_tiles_kernel_with_sort, np_tile_kernels.cu:714-926).
    Returns (rgb [P,3], alpha [P], hits per pixel [P], overflow flag), plus the feature map [P,C] when feat_attr
    is given (render_tiles_kernel_with_sort_and_feat)."""
    ro, rd, geom = _f32(rays_o), _f32(rays_d_unit), _f32(geom)
    off, sp = _i32(tile_offsets), _i32(prims)
    W1, b1, W2, b2, W3, b3 = [_f32(w) for w in weights]
    freq, att = _f32(freq), _f32(att)
    mlp = _Mlp(_p(W1), _p(b1), _p(W2), _p(b2), _p(W3), _p(b3), _p(freq), _p(att),
               freq.size, W1.shape[1], 12 * freq.size, precision)
    P = W * H
    rgb = np.zeros((P, 3), np.float32)
    alpha = np.zeros(P, np.float32)
    hits = np.zeros(P, np.int32)
    ovf = C.c_int32(0)
    fa = feat = None
    S = Cf = 0
    if feat_attr is not None:
        fa = _f32(feat_attr)
        if fa.ndim == 2:
            fa = fa[:, None, :]
        fa = np.ascontiguousarray(fa)
        S, Cf = fa.shape[1], fa.shape[2]
        feat = np.zeros((P, Cf), np.float32)
    lib().orc_render_per_pixel(_p(ro), _p(rd), _p(geom), C.c_int(geom.shape[0]), _p(off, C.c_int32), _p(sp, C.c_int32),
                               C.c_int(W), C.c_int(H), C.c_int(tile), C.c_float(thr), C.byref(mlp), _p(rgb), _p(alpha),
                               _p(hits, C.c_int32), C.byref(ovf), _p(fa), C.c_int(S), C.c_int(Cf), C.c_float(beta),
                               C.c_float(tau), _p(feat))
    if feat_attr is not None:
        return rgb, alpha, hits, bool(ovf.value), feat
    return rgb, alpha, hits, bool(ovf.value)


def bf16_round(x):
    """float32 -> bfloat16 -> float32, round to nearest even (NaN kept)."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = r.view(np.float32).copy()
    out[np.isnan(a)] = np.nan
    return out.reshape(a.shape)


def grouped_weight_gradients_model(offsets, x6, d3, masks, freq, att, weights, dtype="float16", scale=None):
    """Mixed-precision statement of grouped_weight_gradients (scannet/primitive_gemm.py:101-166, the Triton kernel's
    arithmetic): encoding, weights, activations and adjoints rounded to the operand format, FP32 products and sums,
    adjoints scaled before the cast and the sums unscaled afterwards.  dtype "float32" is the unrounded statement
    (scannet/primitive_csr.py:33-58).  masks [R,2] int32 (saved activation signs) or None (signs of the recomputed
    activations, primitive_gemm.py:149-151).  Returns [dW1, db1, dW2, db2, dW3, db3] as float32 arrays."""
    q = {"float32": lambda a: np.asarray(a, np.float32),
         "float16": lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32),     # round to nearest even
         "bfloat16": bf16_round}[dtype]
    if scale is None:
        scale = 4096.0 if dtype == "float16" else 1.0
    W1, b1, W2, b2, W3, b3 = [np.asarray(w, np.float32) for w in weights]
    n = W1.shape[0]
    mult = (np.asarray(freq, np.float32) * np.asarray(att, np.float32)).astype(np.float32)
    out = [np.zeros_like(w) for w in (W1, b1, W2, b2, W3, b3)]
    bit = (1 << np.arange(32, dtype=np.int64))
    for p in range(n):
        b, e = int(offsets[p]), int(offsets[p + 1])
        if b == e:
            continue
        ph = (np.asarray(x6[b:e], np.float32)[:, :, None] * mult[None, None, :]).astype(np.float32)
        enc = q(np.concatenate((np.sin(ph).reshape(e - b, -1), np.cos(ph).reshape(e - b, -1)), axis=1).astype(np.float32))
        w1, w2, w3 = q(W1[p]), q(W2[p]), q(W3[p])
        h1f = (enc.astype(np.float64) @ w1.T.astype(np.float64)).astype(np.float32) + b1[p]
        h1 = q(np.maximum(h1f, 0.0).astype(np.float32))
        h2f = (h1.astype(np.float64) @ w2.T.astype(np.float64)).astype(np.float32) + b2[p]
        h2 = q(np.maximum(h2f, 0.0).astype(np.float32))
        if masks is None:
            a1, a2 = h1f > 0, h2f > 0
        else:
            m = np.asarray(masks[b:e]).astype(np.int64) & 0xFFFFFFFF
            a1, a2 = (m[:, 0:1] & bit[None, :]) != 0, (m[:, 1:2] & bit[None, :]) != 0
        d3q = q((np.asarray(d3[b:e], np.float32) * np.float32(scale)).astype(np.float32))
        d2 = q(((d3q.astype(np.float64) @ w3.astype(np.float64)).astype(np.float32) * a2).astype(np.float32))
        d1 = q(((d2.astype(np.float64) @ w2.astype(np.float64)).astype(np.float32) * a1).astype(np.float32))
        inv = 1.0 / scale
        out[0][p] = (d1.T.astype(np.float64) @ enc.astype(np.float64) * inv).astype(np.float32)
        out[1][p] = (d1.astype(np.float64).sum(0) * inv).astype(np.float32)
        out[2][p] = (d2.T.astype(np.float64) @ h1.astype(np.float64) * inv).astype(np.float32)
        out[3][p] = (d2.astype(np.float64).sum(0) * inv).astype(np.float32)
        out[4][p] = (d3q.T.astype(np.float64) @ h2.astype(np.float64) * inv).astype(np.float32)
        out[5][p] = (d3q.astype(np.float64).sum(0) * inv).astype(np.float32)
    return out
