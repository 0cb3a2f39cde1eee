"""Grouped per-primitive evaluator, same module surface as scannet/primitive_gemm.py.

`GroupLayout`, `prepare_groups` and `resolve_groups` keep the reference's fields, checks and
error texts (primitive_gemm.py:21-52, 186-212).  The reference's only grouped kernel is the
backward VJP (Triton); the inference path needs its forward twin, `grouped_forward`: records
grouped by primitive -> (R, G, B, sigma_raw) per record, evaluated per primitive group on the
tcgen05 tensor cores (fp16 operands, FP32 accumulate) or in scalar FP32.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L


@dataclass(frozen=True)
class GroupLayout:
    """Prepared segments bound to their CSR and segment length (primitive_gemm.py:21-52)."""

    primitives: torch.Tensor
    starts: torch.Tensor
    offsets: torch.Tensor
    segment_size: int
    source_offsets: torch.Tensor
    num_records: int
    tensor_versions: tuple

    def __iter__(self):
        return iter((self.primitives, self.starts, self.offsets))

    def validate(self, csr, segment_size):
        if segment_size != self.segment_size:
            raise ValueError(f"Prepared groups use segment_size={self.segment_size}, "
                             f"but the consumer requested {segment_size}")
        if self.source_offsets is not csr.offsets or self.num_records != len(csr.x6):
            raise ValueError("Prepared groups belong to a different CSR layout")
        tensors = (self.source_offsets, self.primitives, self.starts, self.offsets)
        if tuple(t._version for t in tensors) != self.tensor_versions:
            raise ValueError("Prepared groups or their CSR offsets were modified in place")
        return self


def prepare_groups(csr, segment_size=512):
    if not isinstance(segment_size, int) or isinstance(segment_size, bool) or segment_size <= 0:
        raise ValueError("segment_size must be a positive integer")
    if csr.offsets.ndim != 1 or csr.offsets.dtype != torch.int64 or not csr.offsets.is_contiguous():
        raise ValueError("CSR offsets must be contiguous int64")
    if csr.offsets.numel() < 1:
        raise ValueError("CSR offsets must include the initial zero")
    if not csr.offsets.is_cuda:
        raise RuntimeError("prepare_groups runs on a CUDA device; there is no CPU path")
    lib = L.load()
    dev = csr.offsets.device
    n = int(csr.offsets.numel()) - 1
    group_offsets = torch.empty(n + 1, device=dev, dtype=torch.int64)
    total = C.c_int64(0)
    with torch.cuda.device(dev):
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        L.check(lib.mlpsp_prepare_groups(L.ptr(csr.offsets), n, segment_size, L.ptr(group_offsets), None, None, 0,
                                         C.byref(total), st), "mlpsp_prepare_groups")
        G = int(total.value)
        primitives = torch.empty(G, device=dev, dtype=torch.int64)
        starts = torch.empty(G, device=dev, dtype=torch.int64)
        L.check(lib.mlpsp_prepare_groups(L.ptr(csr.offsets), n, segment_size, L.ptr(group_offsets), L.ptr(primitives),
                                         L.ptr(starts), G, C.byref(total), st), "mlpsp_prepare_groups")
    tensors = (csr.offsets, primitives, starts, group_offsets)
    return GroupLayout(primitives, starts, group_offsets, segment_size, csr.offsets, len(csr.x6),
                       tuple(t._version for t in tensors))


def resolve_groups(csr, segment_size=512, groups=None):
    """Require metadata when a caller shares groups between consumers (primitive_gemm.py:205-212)."""
    if not isinstance(segment_size, int) or isinstance(segment_size, bool) or segment_size <= 0:
        raise ValueError("segment_size must be a positive integer")
    if groups is None:
        return prepare_groups(csr, segment_size)
    if not isinstance(groups, GroupLayout):
        raise TypeError("groups must be a GroupLayout returned by prepare_groups")
    return groups.validate(csr, segment_size)


@torch.no_grad()
def grouped_forward(csr_offsets, x6, scene, *, dtype=torch.float16):
    """Evaluate every record with its primitive's MLP: returns [R,4] = (R, G, B, sigma_raw).

    csr_offsets: int64 [N+1] (records are primitive-major, as group_records lays them out);
    x6: float32 [R,6]; scene: engine.PackedScene; dtype float16 (tensor cores) or float32 (scalar).
    """
    if dtype not in (torch.float32, torch.float16):
        raise ValueError("unsupported GEMM operand dtype")
    if csr_offsets.dtype != torch.int64 or not csr_offsets.is_contiguous() or csr_offsets.numel() != scene.n + 1:
        raise ValueError("CSR offsets and all master tensors must have the same primitive count")
    if x6.ndim != 2 or x6.shape[1] != 6 or x6.dtype != torch.float32:
        raise ValueError("CSR inputs must have shape (records,6) and dtype float32")
    if not x6.is_cuda or not x6.is_contiguous() or x6.device != scene.device:
        raise ValueError("all inputs must be contiguous tensors on one CUDA device")
    if dtype == torch.float16 and not scene.has_f16:
        raise ValueError("the scene holds no packed fp16 weights")
    lib = L.load()
    dev = x6.device
    R = int(x6.shape[0])
    out = torch.empty((R, 4), device=dev, dtype=torch.float32)
    nbytes = int(lib.mlpsp_mlp_grouped_scratch_bytes(R, scene.n))
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    status = torch.zeros(L.STATUS_WORDS, device=dev, dtype=torch.int32)
    with torch.cuda.device(dev):
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        prec = L.PRECISION_F16 if dtype == torch.float16 else L.PRECISION_F32
        L.check(lib.mlpsp_mlp_grouped(C.byref(scene.c), prec, L.ptr(csr_offsets), L.ptr(x6), R, L.ptr(out),
                                      L.ptr(scratch), nbytes, L.ptr(status), st), "mlpsp_mlp_grouped")
        bits = int(status[L.ST_BITS].item())
    if bits & L.BIT_TIMEOUT:
        raise RuntimeError("grouped_forward: a device-side wait gave up; results discarded")
    if bits & L.BIT_NUMERIC:
        raise RuntimeError("grouped_forward: non-finite operand or activation in the fp16 evaluator")
    return out
