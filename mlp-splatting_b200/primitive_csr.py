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
