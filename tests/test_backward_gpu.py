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
        if dtype == torch.float32:
            torch.testing.assert_close(g, want, atol=1.e-4 * scale, rtol=3.e-4)     # the reference test's FP32 bound
        else:
            # the reference test's bound for its tensor-core modes (tests/test_primitive_csr.py:128-130)
            relative_l2 = float((g - want).norm() / want.norm().clamp_min(1.e-30))
            assert relative_l2 < (0.01 if dtype == torch.float16 else 0.04), (k, relative_l2)
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


def _random_csr(dev, n, mean_count, seed, d_scale=1.0):
    from mlp_splatting_b200.primitive_csr import PrimitiveCSR
    g = torch.Generator(device="cpu").manual_seed(seed)
    counts = torch.poisson(torch.full((n,), float(mean_count)), generator=g).to(torch.int64)
    counts[::7] = 0
    counts[3] = 1300                                           # several segments and a ragged tail
    offsets = torch.cat((torch.zeros(1, dtype=torch.int64), counts.cumsum(0))).to(dev)
    R = int(offsets[-1])
    x6 = (torch.randn((R, 6), generator=g) * 0.2).to(dev)
    d3 = (torch.randn((R, 4), generator=g) * d_scale).to(dev)
    weights = [(torch.randn((n, *shape), generator=g) * 0.1).to(dev)
               for shape in [(32, 72), (32,), (32, 32), (32,), (4, 32), (4,)]]
    freq = (2.0 ** torch.arange(6, dtype=torch.float32)).to(dev)
    att = torch.exp(-0.5 * freq.square() * 1.0e-4)
    # exact FP32 activation signs, as the record emitter saves them (the reference test builds them the same way)
    masks = torch.zeros((R, 2), device=dev, dtype=torch.int32)
    bit = 1 << torch.arange(32, device=dev, dtype=torch.int64)
    for p in range(n):
        b, e = int(offsets[p]), int(offsets[p + 1])
        if b == e:
            continue
        ph = x6[b:e, :, None] * freq[None, None, :] * att[None, None, :]
        enc = torch.cat((torch.sin(ph).flatten(1), torch.cos(ph).flatten(1)), dim=1)
        h1 = torch.relu(enc @ weights[0][p].T + weights[1][p])
        h2 = torch.relu(h1 @ weights[2][p].T + weights[3][p])
        masks[b:e, 0] = ((h1 > 0) * bit).sum(1).to(torch.int32)
        masks[b:e, 1] = ((h2 > 0) * bit).sum(1).to(torch.int32)
    return PrimitiveCSR(offsets, torch.arange(R, device=dev), x6, d3, masks), freq, att, weights


@pytest.mark.parametrize("dtype,bound", [(torch.float16, 0.01), (torch.bfloat16, 0.04)])
@pytest.mark.parametrize("segment_size", [512, 128, 32])
def test_tensor_core_gradients_match_fp32_kernel(dtype, bound, segment_size):
    """binary16 / bfloat16 operands on tcgen05 against this library's IEEE FP32 kernel on 300 primitives with ragged
    record counts and saved activation signs, within the reference test's bounds; without saved signs (they are then
    taken from the rounded-operand activations, primitive_gemm.py:149-151, and a few flip) within three times those."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mlp_splatting_b200.primitive_gemm import get_grouped_vjp_safety_stats, grouped_weight_gradients
    dev = torch.device("cuda", 0)
    csr, freq, att, weights = _random_csr(dev, 300, 90, 5)
    before = get_grouped_vjp_safety_stats()
    want = grouped_weight_gradients(csr, freq, att, weights, dtype=torch.float32, segment_size=segment_size)
    got = grouped_weight_gradients(csr, freq, att, weights, dtype=dtype, segment_size=segment_size)
    again = grouped_weight_gradients(csr, freq, att, weights, dtype=dtype, segment_size=segment_size)
    after = get_grouped_vjp_safety_stats()
    assert after["fp32_fallbacks"] == before["fp32_fallbacks"] and after["mixed_calls"] == before["mixed_calls"] + 2
    counts = csr.offsets[1:] - csr.offsets[:-1]
    for g, w, a, k in zip(got, want, again, ("W1", "b1", "W2", "b2", "W3", "b3")):
        assert torch.isfinite(g).all() and torch.equal(g, a)              # deterministic
        relative_l2 = float((g - w).norm() / w.norm())
        assert relative_l2 < bound, (k, relative_l2)
        # per primitive too: no primitive's gradient may be off as a whole
        num = (g - w).flatten(1).norm(dim=1)
        den = w.flatten(1).norm(dim=1).clamp_min(1e-20)
        assert float((num / den)[counts > 0].max()) < 4 * bound, k
        assert (g[counts == 0] == 0).all()
    from mlp_splatting_b200.primitive_csr import PrimitiveCSR
    bare = PrimitiveCSR(csr.offsets, csr.record_indices, csr.x6, csr.grad4, None)
    got = grouped_weight_gradients(bare, freq, att, weights, dtype=dtype, segment_size=segment_size)
    for g, w, k in zip(got, want, ("W1", "b1", "W2", "b2", "W3", "b3")):
        relative_l2 = float((g - w).norm() / w.norm())
        assert relative_l2 < 3 * bound, (k, relative_l2)


@pytest.mark.parametrize("dtype,name,bound", [(torch.float16, "float16", 3e-4), (torch.bfloat16, "bfloat16", 2e-3)])
def test_tensor_core_gradients_match_operand_model(dtype, name, bound):
    """The tcgen05 kernel against the CPU statement of the mixed-precision arithmetic (operands rounded to the format,
    FP32 sums): what is left between the two is the order of the FP32 sums and the rare encoding entry that the
    hardware sine rounds to the neighbouring operand value -- an order of magnitude below the distance to FP32."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import oracle as orc
    from mlp_splatting_b200.primitive_gemm import grouped_weight_gradients
    dev = torch.device("cuda", 0)
    csr, freq, att, weights = _random_csr(dev, 120, 70, 21)
    got = grouped_weight_gradients(csr, freq, att, weights, dtype=dtype, segment_size=128)
    cpu = lambda t: t.detach().cpu().numpy()
    want = orc.grouped_weight_gradients_model(cpu(csr.offsets), cpu(csr.x6), cpu(csr.grad4), cpu(csr.relu_masks), cpu(freq),
                                              cpu(att), [cpu(w) for w in weights], dtype=name)
    f32 = orc.grouped_weight_gradients_model(cpu(csr.offsets), cpu(csr.x6), cpu(csr.grad4), cpu(csr.relu_masks), cpu(freq),
                                             cpu(att), [cpu(w) for w in weights], dtype="float32")
    for g, w, f, k in zip(got, want, f32, ("W1", "b1", "W2", "b2", "W3", "b3")):
        rel = float(np.linalg.norm(cpu(g) - w) / np.linalg.norm(w))
        to_f32 = float(np.linalg.norm(w - f) / np.linalg.norm(f))
        print(name, k, "kernel vs operand model", f"{rel:.2e}", "operand model vs FP32", f"{to_f32:.2e}")
        assert rel < bound and rel < to_f32, (k, rel, to_f32)


def test_nonfinite_mixed_result_is_retried_in_fp32():
    """Adjoints that overflow binary16 once scaled by 4096: the mixed launch raises the flag, the call warns, retries
    in unscaled IEEE FP32 and returns that result (primitive_gemm.py:64-98)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mlp_splatting_b200.primitive_gemm import get_grouped_vjp_safety_stats, grouped_weight_gradients
    dev = torch.device("cuda", 0)
    csr, freq, att, weights = _random_csr(dev, 40, 60, 9, d_scale=100.0)      # 100 * 4096 > 65504
    want = grouped_weight_gradients(csr, freq, att, weights, dtype=torch.float32)
    before = get_grouped_vjp_safety_stats()["fp32_fallbacks"]
    with pytest.warns(RuntimeWarning, match="retrying with IEEE FP32"):
        got = grouped_weight_gradients(csr, freq, att, weights, dtype=torch.float16)
    assert get_grouped_vjp_safety_stats()["fp32_fallbacks"] == before + 1
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    # bfloat16 has the range: no retry, result within its bound
    got = grouped_weight_gradients(csr, freq, att, weights, dtype=torch.bfloat16)
    assert get_grouped_vjp_safety_stats()["fp32_fallbacks"] == before + 1
    assert float((got[0] - want[0]).norm() / want[0].norm()) < 0.04


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
