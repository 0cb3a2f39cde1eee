"""Grouped per-primitive evaluator, same module surface as scannet/primitive_gemm.py.

`GroupLayout`, `prepare_groups` and `resolve_groups` keep the reference's fields, checks and
error texts (primitive_gemm.py:21-52, 186-212).  The reference's only grouped kernel is the
backward VJP (Triton); the inference path needs its forward twin, `grouped_forward`: records
grouped by primitive -> (R, G, B, sigma_raw) per record, evaluated per primitive group on the
tcgen05 tensor cores (fp16 operands, FP32 accumulate) or in scalar FP32.  `grouped_weight_gradients`
is the VJP itself: IEEE FP32, or binary16 / bfloat16 operands on the tensor cores with the reference's
loss scale and FP32 retry.
"""
from __future__ import annotations

import ctypes as C
import warnings
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


# ---- grouped backward: per-primitive weight gradients (scannet/primitive_gemm.py:52-279) ----
_SAFETY_STATS = {"calls": 0, "mixed_calls": 0, "fp32_fallbacks": 0, "fp32_nonfinite_failures": 0}


def get_grouped_vjp_safety_stats(*, reset=False):
    """Process-local counters for run reports; resetting is explicit (primitive_gemm.py:55-62)."""
    snapshot = dict(_SAFETY_STATS)
    if reset:
        for key in _SAFETY_STATS:
            _SAFETY_STATS[key] = 0
    return snapshot


def _checked_grouped_vjp(launch, dtype, loss_scale):
    """Never hand a non-finite MLP gradient to the caller's optimizer step (primitive_gemm.py:64-98): a finite
    result is returned unchanged; a non-finite mixed-precision result is recomputed in unscaled IEEE FP32 from the
    same masters and masks; a non-finite FP32 result raises and returns nothing."""
    _SAFETY_STATS["calls"] += 1
    mixed = dtype != torch.float32
    _SAFETY_STATS["mixed_calls"] += int(mixed)
    result, nonfinite = launch(dtype, loss_scale)
    if not nonfinite:
        return result
    if mixed:
        _SAFETY_STATS["fp32_fallbacks"] += 1
        warnings.warn(
            f"[CSR safety] Nonfinite {dtype} MLP VJP; retrying with IEEE FP32 "
            f"before Adam (FP32 fallbacks={_SAFETY_STATS['fp32_fallbacks']}).",
            RuntimeWarning, stacklevel=3)
        result, nonfinite = launch(torch.float32, 1.0)
        if not nonfinite:
            return result
    _SAFETY_STATS["fp32_nonfinite_failures"] += 1
    raise FloatingPointError(
        "[CSR safety] IEEE FP32 MLP VJP is nonfinite; no gradients were returned "
        "and Adam must not step. Inspect the saved model, records and loss. "
        f"Safety counters: {get_grouped_vjp_safety_stats()}")


@torch.no_grad()
def grouped_weight_gradients(csr, freq, attenuation, weights, *, dtype=torch.float16, segment_size=512, block_size=32,
                             loss_scale=None, groups=None):
    """[dW1, db1, dW2, db2, dW3, db3] of the 72->32->32->4 per-primitive MLP from primitive-major records.

    Same arguments, checks, error texts and safety policy as the reference function (primitive_gemm.py:236-279).
    float32 is IEEE FP32 on the CUDA cores; float16 / bfloat16 round the operands (encoding, activations, adjoints,
    weights) to that format and run every product on the tensor cores with FP32 accumulation over the segment;
    float16 adjoints are scaled by 4096 before the cast and unscaled in FP32 afterwards unless loss_scale says
    otherwise.  A non-finite mixed result is retried in unscaled FP32; a non-finite FP32 result raises
    FloatingPointError and no gradients are returned.  block_size is the reference's Triton row block; it is
    checked and otherwise unused (the kernels walk a segment 128 records at a time)."""
    import math
    w1, b1, w2, b2, w3, b3 = weights
    n = len(w1)
    if [tuple(w.shape[1:]) for w in weights] != [(32, 72), (32,), (32, 32), (32,), (4, 32), (4,)]:
        raise ValueError("grouped backward requires the 72→32→32→4 architecture")
    if any(len(w) != n for w in weights) or csr.offsets.numel() != n + 1:
        raise ValueError("CSR offsets and all master tensors must have the same primitive count")
    if csr.x6.ndim != 2 or csr.x6.shape[1] != 6 or csr.grad4.shape != (len(csr.x6), 4):
        raise ValueError("CSR inputs/adjoints must have shapes (records,6) and (records,4)")
    if freq.numel() != 6 or attenuation.numel() != 6:
        raise ValueError("grouped backward requires six positional frequencies")
    if dtype not in [torch.float32, torch.float16, torch.bfloat16]:
        raise ValueError("unsupported GEMM operand dtype")
    if block_size not in (32, 64) or segment_size <= 0 or segment_size % block_size:
        raise ValueError("segment size must be a positive multiple of the 32/64-row block")
    for tensor in [csr.offsets, csr.x6, csr.grad4, freq, attenuation, *weights]:
        if not tensor.is_cuda or not tensor.is_contiguous() or tensor.device != w1.device:
            raise ValueError("all inputs must be contiguous tensors on one CUDA device")
    if any(t.dtype != torch.float32 for t in [csr.x6, csr.grad4, freq, attenuation, *weights]):
        raise ValueError("master weights, records and encoding parameters must be FP32")
    if csr.relu_masks is not None and (
            csr.relu_masks.dtype != torch.int32 or not csr.relu_masks.is_contiguous()
            or csr.relu_masks.device != w1.device or csr.relu_masks.shape != (len(csr.x6), 2)):
        raise ValueError("saved ReLU masks must be contiguous CUDA int32 with shape (records,2)")
    groups = resolve_groups(csr, segment_size, groups)
    scale = float(4096 if dtype == torch.float16 else 1) if loss_scale is None else float(loss_scale)
    if not math.isfinite(scale) or scale <= 0:
        raise ValueError("loss_scale must be finite and strictly positive")
    lib = L.load()
    dev = w1.device
    glen = int(lib.mlpsp_grouped_gradient_floats())
    G = int(groups.primitives.numel())
    sc = L.Scene()
    sc.n, sc.hidden, sc.num_freq = n, 32, 6
    sc.W1, sc.b1, sc.W2, sc.b2, sc.W3, sc.b3 = (L.ptr(t) for t in weights)
    sc.freq, sc.att = L.ptr(freq), L.ptr(attenuation)
    precisions = {torch.float32: L.PRECISION_F32, torch.float16: L.PRECISION_F16, torch.bfloat16: L.PRECISION_BF16}

    def launch(operand_dtype, operand_scale):
        """One unguarded launch, shared by the normal path and the FP32 retry (primitive_gemm.py:215-232)."""
        partial = torch.empty((max(G, 1), glen), device=dev, dtype=torch.float32)
        result = torch.empty((n, glen), device=dev, dtype=torch.float32)
        nonfinite = torch.zeros((), device=dev, dtype=torch.int32)
        with torch.cuda.device(dev):
            st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            L.check(lib.mlpsp_grouped_weight_gradients(
                C.byref(sc), L.ptr(csr.offsets), L.ptr(csr.x6), L.ptr(csr.grad4), L.ptr(csr.relu_masks),
                L.ptr(groups.primitives), L.ptr(groups.starts), L.ptr(groups.offsets), G, int(segment_size),
                precisions[operand_dtype], float(operand_scale), L.ptr(partial), L.ptr(result), L.ptr(nonfinite), st),
                "mlpsp_grouped_weight_gradients")
        word = int(nonfinite.item())
        if word & 2:
            raise RuntimeError("grouped_weight_gradients: a device-side wait gave up; results discarded")
        return result, bool(word & 1)

    result = _checked_grouped_vjp(launch, dtype, scale)
    sizes = [2304, 32, 1024, 32, 128, 4]
    return [v.reshape(w.shape).contiguous() for v, w in zip(result.split(sizes, dim=1), weights)]
