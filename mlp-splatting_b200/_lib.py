"""ctypes binding of libmlpsp_b200.so (the C ABI declared in include/mlpsp.h).

There is no fallback: if the shared library is missing or cannot be loaded, every use of the
render path raises.  Build it with `python mlp-splatting_b200/build.py`.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmlpsp_b200.so")

STATUS_WORDS = 16
ST_BITS, ST_MAX_TILE_LEN, ST_PAIRS, ST_WAVES = 0, 1, 2, 3
ST_RECORDS_LO, ST_USED_LO, ST_WAVE_RECORDS, ST_WORK_ITEMS, ST_WORK_TOTAL, ST_PAIRS_KEPT, ST_WORK_SMALL = 4, 6, 8, 9, 10, 11, 12
BIT_BAD_OFFSETS, BIT_TILE_CAPACITY, BIT_BAD_IDS = 1, 2, 4
BIT_PAIR_OVERFLOW, BIT_RECORD_OVERFLOW, BIT_NUMERIC, BIT_TIMEOUT = 8, 16, 64, 128
BIT_TILE_ORIGINS, BIT_CONE_TOO_WIDE, BIT_FEAT_INEXACT = 256, 512, 1024
BIT_PIXEL_HITS = 32
ORDER_PER_PIXEL = 2
PRECISION_F32, PRECISION_F16, PRECISION_BF16 = 0, 1, 2
MAX_WAVES = 32
GEOM_FLOATS = 16
KERNEL_CLASSES = ("bin", "sort", "hits", "prim_scan", "fill", "mlp", "composite", "other")

_fp = C.c_void_p  # device or host pointers travel as plain addresses


class Scene(C.Structure):
    _fields_ = [
        ("geom", _fp), ("n", C.c_int32), ("hidden", C.c_int32), ("num_freq", C.c_int32), ("reserved0", C.c_int32),
        ("W1", _fp), ("b1", _fp), ("W2", _fp), ("b2", _fp), ("W3", _fp), ("b3", _fp),
        ("w16", _fp), ("freq", _fp), ("att", _fp), ("feat_attr", _fp),
        ("feat_slots", C.c_int32), ("feat_dim", C.c_int32), ("gate_beta", C.c_float), ("gate_tau", C.c_float),
        ("wbf16", _fp), ("feat16", _fp),
    ]


class Frame(C.Structure):
    _fields_ = [
        ("rays_o", _fp), ("rays_d", _fp),
        ("width", C.c_int32), ("height", C.c_int32), ("tile", C.c_int32), ("threshold", C.c_float),
        ("tile_capacity", C.c_int32), ("precision", C.c_int32),
        ("view", _fp), ("proj", _fp),
        ("tile_offsets", _fp), ("tile_prims", _fp), ("sorted_prims", _fp), ("max_pairs", C.c_int64),
        ("rgb", _fp), ("alpha", _fp), ("depth_t", _fp), ("feat", _fp), ("mask_used", _fp), ("bg_color", _fp),
        ("scratch", _fp), ("scratch_bytes", C.c_int64), ("max_records", C.c_int64),
        ("status", _fp), ("num_waves", C.c_int32), ("wave_len", C.c_int32 * MAX_WAVES),
        ("keep_records", C.c_int32), ("sort_key", C.c_int32),
        ("tile_row_begin", C.c_int32), ("tile_row_end", C.c_int32),
        ("tile_pretest", C.c_int32), ("tail_hint", C.c_int32),
        ("gt_rgb", _fp), ("stat_sum_w", _fp), ("stat_max_w", _fp), ("stat_hits", _fp), ("stat_sum_werr", _fp),
        ("stat_contrib", _fp),
        ("hit_arith", C.c_int32), ("reserved1", C.c_int32),
    ]


class Decoder(C.Structure):
    _fields_ = [("in_dim", C.c_int32), ("hidden", C.c_int32), ("out_dim", C.c_int32), ("num_classes", C.c_int32),
                ("W1", _fp), ("b1", _fp), ("W2", _fp), ("b2", _fp), ("W3", _fp), ("b3", _fp), ("text", _fp)]


_SIGS = {
    "mlpsp_last_error": (C.c_char_p, []),
    "mlpsp_abi_version": (C.c_int, []),
    "mlpsp_struct_sizes": (C.c_int, [C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "mlpsp_pack_geometry": (C.c_int, [_fp, _fp, _fp, C.c_int32, _fp, _fp]),
    "mlpsp_normalize_rows": (C.c_int, [_fp, _fp, C.c_int64, C.c_int32, _fp]),
    "mlpsp_packed_weight_bytes": (C.c_int64, [C.c_int32, C.c_int32]),
    "mlpsp_pack_weights_f16": (C.c_int, [C.POINTER(Scene), _fp, _fp, _fp]),
    "mlpsp_pack_weights_bf16": (C.c_int, [C.POINTER(Scene), _fp, _fp, _fp]),
    "mlpsp_pack_features_f16": (C.c_int, [C.POINTER(Scene), _fp, _fp, _fp]),
    "mlpsp_records_reverse": (C.c_int, [_fp, _fp, _fp, _fp, _fp, _fp, _fp, _fp, C.c_int64, C.c_int64, C.c_int32, _fp, _fp, _fp, _fp, _fp]),
    "mlpsp_grouped_gradient_floats": (C.c_int64, []),
    "mlpsp_grouped_weight_gradients": (C.c_int, [C.POINTER(Scene), _fp, _fp, _fp, _fp, _fp, _fp, _fp, C.c_int64, C.c_int32,
                                                 C.c_int32, C.c_float, _fp, _fp, _fp, _fp]),
    "mlpsp_decoder_packed_bytes": (C.c_int64, [C.POINTER(Decoder), C.c_int32]),
    "mlpsp_pack_decoder": (C.c_int, [C.POINTER(Decoder), C.c_int32, _fp, _fp, _fp]),
    "mlpsp_decode_features": (C.c_int, [C.POINTER(Decoder), C.c_int32, _fp, _fp, C.c_int32, C.c_int32, _fp, _fp, _fp, _fp]),
    "mlpsp_classify_features": (C.c_int, [_fp, C.c_int64, C.c_int32, _fp, C.c_int32, _fp, _fp]),
    "mlpsp_status_reset": (C.c_int, [_fp, _fp]),
    "mlpsp_kernel_launches": (C.c_int, [C.POINTER(C.c_int64), C.c_int32]),
    "mlpsp_timing_enable": (C.c_int, [C.c_int32]),
    "mlpsp_timing_collect": (C.c_int, [C.POINTER(C.c_float), C.c_int32]),
    "mlpsp_frame_scratch_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64]),
    "mlpsp_bin_tiles": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp]),
    "mlpsp_bin_tiles_mosaic": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp, _fp, C.c_int32, _fp]),
    "mlpsp_bin_tiles_raycone": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp]),
    "mlpsp_validate_tile_lists": (C.c_int, [_fp, _fp, C.c_int32, C.c_int64, C.c_int32, C.c_int32, _fp, _fp]),
    "mlpsp_sort_tiles": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp, _fp]),
    "mlpsp_hit_masks": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp, _fp]),
    "mlpsp_render_sorted": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp]),
    "mlpsp_render_frames": (C.c_int, [C.POINTER(Scene), _fp, C.c_int32, _fp]),
    "mlpsp_render_frame": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp]),
    "mlpsp_export_records": (C.c_int, [C.POINTER(Scene), C.POINTER(Frame), _fp, _fp, _fp, _fp, _fp, _fp, C.c_int64,
                                       C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int32), _fp]),
    "mlpsp_mlp_grouped_scratch_bytes": (C.c_int64, [C.c_int64, C.c_int32]),
    "mlpsp_mlp_grouped": (C.c_int, [C.POINTER(Scene), C.c_int32, _fp, _fp, C.c_int64, _fp, _fp, C.c_int64, _fp, _fp]),
    "mlpsp_group_records_scratch_bytes": (C.c_int64, [C.c_int64, C.c_int32]),
    "mlpsp_group_records": (C.c_int, [_fp, C.c_int64, C.c_int32, _fp, _fp, _fp, C.c_int64, _fp]),
    "mlpsp_prepare_groups": (C.c_int, [_fp, C.c_int32, C.c_int64, _fp, _fp, _fp, C.c_int64, C.POINTER(C.c_int64), _fp]),
    "mlpsp_prepare_groups_static": (C.c_int, [_fp, C.c_int32, C.c_int64, _fp, _fp, _fp, C.c_int64, C.POINTER(C.c_int64), _fp]),
}

EXPORTS = tuple(_SIGS)

_lib = None


def load():
    """Load the shared library once; raise with the build command when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(run `python mlp-splatting_b200/build.py`). There is no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        if lib.mlpsp_abi_version() != 1:
            raise RuntimeError("libmlpsp_b200.so ABI version mismatch; rebuild it")
        a, b = C.c_int32(0), C.c_int32(0)
        lib.mlpsp_struct_sizes(C.byref(a), C.byref(b))
        if (a.value, b.value) != (C.sizeof(Scene), C.sizeof(Frame)):
            raise RuntimeError("mlpsp_scene/mlpsp_frame layout differs between the library and its binding")
        _lib = lib
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().mlpsp_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed ({rc}): {msg}")


def ptr(t):
    """Address of a torch tensor's storage (None -> NULL)."""
    return None if t is None else t.data_ptr()
