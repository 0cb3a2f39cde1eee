"""Backward side of the record path against tests/golden/backward.npz (made by tests/golden/make_golden.py):
per-primitive weight gradients from the reference's own PyTorch statement (scannet/primitive_csr.py:33-58) on the
record counts of its test (tests/test_primitive_csr.py:91-134), and reverse-compositing adjoints from torch autograd;
plus the reference's primitive_records_reverse kernel itself where oracle/_ref has been built."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def fx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return np.load(os.path.join(HERE, "golden", "backward.npz"))


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("scale", [1.0, 1.0e-6])
@pytest.mark.parametrize("segment_size", [512, 64])
def test_grouped_weight_gradients_match_reference_statement(fx, dtype, scale, segment_size):
    from mlp_splatting_b200.primitive_csr import PrimitiveCSR
    from mlp_splatting_b200.primitive_gemm import grouped_weight_gradients, prepare_groups
    dev = torch.device("cuda", 0)
    R = fx["vjp_x6"].shape[0]
    csr = PrimitiveCSR(_t(fx["vjp_offsets"], dev), torch.arange(R, device=dev), _t(fx["vjp_x6"], dev),
                       _t(fx["vjp_d3"], dev) * scale, _t(fx["vjp_masks"], dev))
    weights = [_t(fx["vjp_" + k], dev) for k in ("W1", "b1", "W2", "b2", "W3", "b3")]
    groups = prepare_groups(csr, segment_size)
    got = grouped_weight_gradients(csr, _t(fx["vjp_freq"], dev), _t(fx["vjp_att"], dev), weights, dtype=dtype,
                                   segment_size=segment_size, groups=groups)
    for g, k in zip(got, ("W1", "b1", "W2", "b2", "W3", "b3")):
        want = _t(fx["vjp_g" + k], dev) * scale
        assert torch.isfinite(g).all()
        torch.testing.assert_close(g, want, atol=1.e-4 * scale, rtol=3.e-4)     # the reference test's FP32 bound
        for empty in (0, 9):
            assert (g[empty] == 0).all()
    # without saved masks the signs are recomputed: same result on this data
    csr2 = PrimitiveCSR(csr.offsets, csr.record_indices, csr.x6, csr.grad4, None)
    again = grouped_weight_gradients(csr2, _t(fx["vjp_freq"], dev), _t(fx["vjp_att"], dev), weights, dtype=torch.float32,
                                     segment_size=segment_size)
    torch.testing.assert_close(again[0], _t(fx["vjp_gW1"], dev) * scale, atol=1.e-4 * scale, rtol=3.e-4)


def test_grouped_weight_gradients_errors(fx):
    from mlp_splatting_b200.primitive_csr import PrimitiveCSR
    from mlp_splatting_b200.primitive_gemm import get_grouped_vjp_safety_stats, grouped_weight_gradients
    dev = torch.device("cuda", 0)
    R = fx["vjp_x6"].shape[0]
    csr = PrimitiveCSR(_t(fx["vjp_offsets"], dev), torch.arange(R, device=dev), _t(fx["vjp_x6"], dev),
                       _t(fx["vjp_d3"], dev), None)
    weights = [_t(fx["vjp_" + k], dev) for k in ("W1", "b1", "W2", "b2", "W3", "b3")]
    freq, att = _t(fx["vjp_freq"], dev), _t(fx["vjp_att"], dev)
    with pytest.raises(ValueError, match="segment size must be a positive multiple"):
        grouped_weight_gradients(csr, freq, att, weights, segment_size=100)
    with pytest.raises(ValueError, match="unsupported GEMM operand dtype"):
        grouped_weight_gradients(csr, freq, att, weights, dtype=torch.float64)
    with pytest.raises(ValueError, match="requires the 72"):
        grouped_weight_gradients(csr, freq, att, [weights[0][:, :, :60]] + weights[1:])
    bad = PrimitiveCSR(csr.offsets, csr.record_indices, csr.x6, csr.grad4.clone(), None)
    bad.grad4[5, 0] = float("inf")
    before = get_grouped_vjp_safety_stats()["fp32_nonfinite_failures"]
    with pytest.raises(FloatingPointError, match="MLP VJP is nonfinite"):
        grouped_weight_gradients(bad, freq, att, weights, dtype=torch.float32)
    assert get_grouped_vjp_safety_stats()["fp32_nonfinite_failures"] == before + 1


def test_records_reverse_matches_autograd(fx):
    from mlp_splatting_b200.primitive_csr import primitive_records_reverse
    dev = torch.device("cuda", 0)
    d4, gp, gs, gq = primitive_records_reverse(_t(fx["rev_ids"], dev), _t(fx["rev_offsets"], dev), _t(fx["rev_x6"], dev),
                                               _t(fx["rev_raw"], dev), _t(fx["rev_logs"], dev), _t(fx["rev_quats"], dev),
                                               _t(fx["rev_grgb"], dev), _t(fx["rev_gt"], dev))
    for got, key in ((d4, "rev_d4"), (gp, "rev_gp"), (gs, "rev_gs"), (gq, "rev_gq")):
        want = _t(fx[key], dev)
        torch.testing.assert_close(got, want, atol=2e-5 * float(want.abs().max()) + 1e-7, rtol=2e-4)
    assert float(_t(fx["rev_gq"], dev).abs().max()) > 1e-4       # the quaternion path is exercised


def test_records_reverse_matches_reference_kernel():
    """primitive_records_reverse of the reference extension on records exported by this library."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import build_ref
    ref = build_ref.load_module()
    if ref is None:
        pytest.skip("reference extension not built (python oracle/build_ref.py)")
    from mlp_splatting_b200.engine import normalize_rows
    from mlp_splatting_b200.primitive_csr import primitive_records_reverse
    from tests.helpers import small_case
    from tests.test_parity_gpu import CASES, _packed, _renderer
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES["tiny"])
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    _rgb, _alpha, ids, x6, raw, _masks, _gates, offsets = r.render_records(
        ps, _t(cam["rays_o"], dev), _t(cam["rays_d"], dev), 5e-3, view=cam["view"], proj=cam["proj"], precision=0)
    P = cam["W"] * cam["H"]
    g = torch.Generator(device=dev).manual_seed(11)
    grgb = torch.randn((P, 3), device=dev, generator=g)
    gt = torch.randn((P,), device=dev, generator=g)
    logs = _t(scene["log_scales"], dev)
    quats = normalize_rows(_t(scene["quats"], dev))
    mine = primitive_records_reverse(ids, offsets, x6, raw, logs, quats, grgb, gt)
    theirs = ref.primitive_records_reverse(ids, offsets, x6, raw, logs, quats, grgb, gt)
    assert ids.numel() > 10000
    for a, b in zip(mine, theirs):
        torch.testing.assert_close(a, b, atol=5e-5 * float(b.abs().max()) + 1e-7, rtol=2e-4)
