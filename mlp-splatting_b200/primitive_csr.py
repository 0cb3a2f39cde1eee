"""Primitive-major record grouping, same surface as scannet/primitive_csr.py:14-29.

`group_records` returns the same `PrimitiveCSR` fields; the stable grouping runs as a device-wide
radix sort inside libmlpsp_b200.so instead of torch.argsort/bincount/cumsum.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L


@dataclass
class PrimitiveCSR:
    offsets: torch.Tensor
    record_indices: torch.Tensor
    x6: torch.Tensor
    grad4: torch.Tensor
    relu_masks: torch.Tensor | None = None


def group_order(primitive_ids: torch.Tensor, num_primitives: int):
    """(offsets int64 [N+1], order int64 [R]): records grouped by primitive, record order kept inside a group."""
    lib = L.load()
    if not primitive_ids.is_cuda:
        raise RuntimeError("group_records runs on a CUDA device; there is no CPU path")
    ids = primitive_ids.to(torch.int32).contiguous()
    dev = ids.device
    R, n = int(ids.numel()), int(num_primitives)
    offsets = torch.empty(n + 1, device=dev, dtype=torch.int64)
    order = torch.empty(R, device=dev, dtype=torch.int64)
    nbytes = int(lib.mlpsp_group_records_scratch_bytes(R, n))
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        L.check(lib.mlpsp_group_records(L.ptr(ids), R, n, L.ptr(offsets), L.ptr(order), L.ptr(scratch), nbytes, st),
                "mlpsp_group_records")
    return offsets, order


def group_records(primitive_ids, x6, grad4, num_primitives: int, relu_masks=None) -> PrimitiveCSR:
    """Group records by primitive, preserving pixel order inside each group."""
    offsets, order = group_order(primitive_ids, num_primitives)
    return PrimitiveCSR(offsets, order, x6[order], grad4[order],
                        None if relu_masks is None else relu_masks[order])


@torch.no_grad()
def primitive_records_reverse(ids, offsets, x6, raw, log_scales, quats, grad_rgb, grad_t):
    """Reverse compositing over saved records, the extension entry of the same name in the reference
    (scannet/cuda/primitive_records.cuh:51-74): returns [d4 (R,4), grad_positions (N,3), grad_log_scales (N,3),
    grad_quats (N,4)].  ids int32 [R]; offsets int64 [pixels+1]; x6 [R,6]; raw [R,8]; float32 CUDA tensors."""
    for t in (ids, offsets, x6, raw, log_scales, quats, grad_rgb, grad_t):
        if not (t.is_cuda and t.is_contiguous() and t.device == ids.device):
            raise ValueError("all inputs must be contiguous tensors on one CUDA device")
    if ids.dtype != torch.int32 or offsets.dtype != torch.int64:
        raise ValueError("ids must be int32 and offsets int64")
    if any(t.dtype != torch.float32 for t in (x6, raw, log_scales, quats, grad_rgb, grad_t)):
        raise ValueError("records, geometry and adjoints must be FP32")
    total, pixels, n = int(ids.numel()), int(grad_rgb.shape[0]), int(log_scales.shape[0])
    if offsets.ndim != 1 or offsets.numel() != pixels + 1 or x6.shape != (total, 6) or raw.shape != (total, 8):
        raise ValueError("record tensors do not match the pixel offsets")
    if quats.shape != (n, 4) or log_scales.shape != (n, 3) or grad_rgb.shape != (pixels, 3) or grad_t.numel() != pixels:
        raise ValueError("geometry or adjoint shapes do not match")
    if int(offsets[0]) != 0 or int(offsets[-1]) != total or bool((offsets[1:] < offsets[:-1]).any()):
        raise ValueError("pixel offsets must start at zero, end at the record count and be monotone")
    if total and (int(ids.min()) < 0 or int(ids.max()) >= n):
        raise ValueError("record primitive ids out of range")
    lib = L.load()
    dev = ids.device
    d4 = torch.empty((total, 4), device=dev, dtype=torch.float32)
    gp = torch.empty((n, 3), device=dev, dtype=torch.float32)
    gs = torch.empty((n, 3), device=dev, dtype=torch.float32)
    gq = torch.empty((n, 4), device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        L.check(lib.mlpsp_records_reverse(L.ptr(ids), L.ptr(offsets), L.ptr(x6), L.ptr(raw), L.ptr(log_scales), L.ptr(quats),
                                          L.ptr(grad_rgb), L.ptr(grad_t), pixels, total, n, L.ptr(d4), L.ptr(gp), L.ptr(gs),
                                          L.ptr(gq), st), "mlpsp_records_reverse")
    return [d4, gp, gs, gq]
