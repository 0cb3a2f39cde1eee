"""GPU-vs-GPU parity against the reference's own CUDA kernels.

oracle/build_ref.py compiles the reference's scannet/cuda/np_tile_kernels.cu (unmodified, from its
checkout) into oracle/_ref/mlpsp_ref_ext.so; these tests run its entry points and this library on
the same device, the same tensors and the same tile lists.  They are skipped when the module has
not been built.  Differences that remain are the ones the arithmetic contract predicts: the
reference uses hardware __expf where this library uses an IEEE-only exp, so a decision can flip
where the reference's own value sits within a few ulp of a threshold.
"""
import numpy as np
import pytest
import torch

from tests.helpers import WKEYS, oracle_frame, small_case
from tests.test_parity_gpu import CASES, _packed, _renderer, _t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import build_ref
    mod = build_ref.load_module()
    if mod is None:
        pytest.skip("reference extension not built (python oracle/build_ref.py)")
    return mod


def _inputs(scene, cam, f, dev):
    from mlp_splatting_b200.engine import normalize_rows
    base = [_t(cam["rays_o"], dev), _t(f["rays_d_unit"], dev), _t(scene["positions"], dev), _t(scene["log_scales"], dev),
            normalize_rows(_t(scene["quats"], dev)), _t(f["tile_prims"], dev), _t(f["tile_offsets"], dev),
            _t(scene["freq"], dev), _t(scene["att"], dev)] + [_t(scene[k], dev) for k in WKEYS]
    return base


@pytest.mark.parametrize("name", ["tiny", "ragged"])
def test_tile16_forward_matches_reference_kernel(ref, name):
    """render_tiles_forward_tilecenter with 16x16 tiles (the reference's tile_size = 16, scalar kernels) on lists
    culled per 16x16 tile, against render_tile16: 8x8 tiles that inherit the 16x16 tile's ordered list."""
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES[name])
    f = oracle_frame(scene, cam, 5e-3, precision=0, tile=16, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    rgb_r, alpha_r = ref.render_tiles_forward_tilecenter(*x, cam["W"], cam["H"], 16, 16, 5e-3)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    rgb, alpha = r.render_tile16(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True)
    d_rgb = (rgb - rgb_r).abs().max().item()
    d_a = (alpha - alpha_r).abs().max().item()
    assert d_rgb <= 1e-4 and d_a <= 1e-4, (d_rgb, d_a)
    assert alpha_r.mean().item() > 0.05


@pytest.mark.parametrize("name", ["tiny", "ragged", "dense"])
def test_fp32_forward_matches_reference_kernel(ref, name):
    """render_tiles_forward_tilecenter (np_tile_kernels.cu:5225) vs the FP32 path of this library."""
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES[name])
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    rgb_r, alpha_r = ref.render_tiles_forward_tilecenter(*x, cam["W"], cam["H"], 8, 8, 5e-3)
    rgb_t, alpha_t, t_r = ref.render_tiles_forward_tilecenter_with_t(*x, cam["W"], cam["H"], 8, 8, 5e-3)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    rgb, alpha = r.render(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True)
    d_rgb = (rgb - rgb_r).abs().max().item()
    d_a = (alpha - alpha_r).abs().max().item()
    assert d_rgb <= 1e-4 and d_a <= 1e-4, (d_rgb, d_a)
    # the reference's expected-depth kernel sorts by Euclidean depth on the tile-centre ray
    # (np_tile_kernels.cu:5538-5543): sort_key=1 reproduces its rgb, alpha and t
    rgb2, alpha2 = r.render(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True,
                            want_depth=True, sort_key=1)
    assert (rgb2 - rgb_t).abs().max().item() <= 1e-4 and (alpha2 - alpha_t).abs().max().item() <= 1e-4
    # sum(w t)/sum(w) is ill-conditioned where the whole pixel weight is ~1e-7 (alpha = 1 - exp(-x) is
    # quantised at 6e-8 there), in both implementations: compare it where the pixel has visible coverage
    vis = alpha_t > 1e-3
    assert ((r.depth_t - t_r).abs()[vis]).max().item() <= 1e-3
    assert vis.float().mean().item() > 0.2


@pytest.mark.parametrize("name", ["tiny", "dense"])
def test_fp16_forward_matches_reference_wmma_kernel(ref, name):
    """render_tiles_rgb_wmma (rgb_wmma.cuh:225): the tensor-core kernel this library replaces."""
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES[name])
    f = oracle_frame(scene, cam, 5e-3, precision=1, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    rgb_r, alpha_r = ref.render_tiles_rgb_wmma(x, cam["W"], cam["H"], 5e-3, False)
    ps, r = _packed(scene, dev, pack_f16=True), _renderer(cam, dev)
    rgb, alpha = r.render(ps, x[0], x[1], 5e-3, precision=1, tile_lists=(x[5], x[6]), rays_normalized=True)
    assert (rgb - rgb_r).abs().max().item() <= 2e-3      # the tolerance the path is specified to
    assert (alpha - alpha_r).abs().max().item() <= 2e-3
    assert (rgb - rgb_r).abs().mean().item() <= 5e-5


@pytest.mark.parametrize("name", ["tiny", "ragged", "dense"])
def test_records_and_csr_match_reference_kernel(ref, name):
    """render_tiles_training_records (np_tile_kernels.cu:6994) vs this library's record export."""
    from mlp_splatting_b200 import primitive_csr
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES[name])
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    P = cam["W"] * cam["H"]
    x17 = x + [torch.zeros((P, 3), device=dev), torch.zeros(P, device=dev)]
    ref_out = ref.render_tiles_training_records(x17, cam["W"], cam["H"], 8, 5e-3, 1.5, 2.0)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    out = r.render_records(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True)
    names = ["rgb", "alpha", "ids", "x6", "raw", "masks", "gates", "offsets"]
    R, G = dict(zip(names, [t.cpu().numpy() for t in ref_out])), dict(zip(names, [t.cpu().numpy() for t in out]))
    assert R["offsets"].dtype == G["offsets"].dtype == np.int64 and R["ids"].dtype == G["ids"].dtype
    cr, cg = np.diff(R["offsets"]), np.diff(G["offsets"])
    same = cr == cg
    # per-pixel record lists: identical except where the reference's own arithmetic sits on a threshold
    assert (~same).mean() <= 2e-3, f"{(~same).sum()} of {same.size} pixels differ in record count"
    pr, pg = np.repeat(np.arange(cr.size), cr), np.repeat(np.arange(cg.size), cg)
    sr, sg = same[pr], same[pg]
    ids_equal = R["ids"][sr] == G["ids"][sg]
    assert ids_equal.mean() >= 0.999
    keep = ids_equal
    np.testing.assert_allclose(G["x6"][sg][keep], R["x6"][sr][keep], rtol=0, atol=1e-5)
    np.testing.assert_allclose(G["raw"][sg][keep][:, :3], R["raw"][sr][keep][:, :3], rtol=0, atol=3e-5)
    np.testing.assert_allclose(G["raw"][sg][keep][:, 4:7], R["raw"][sr][keep][:, 4:7], rtol=0, atol=3e-5)
    # gates depend on q = R^T (c - p), a difference of O(1) numbers of size ~1e-2: relative 1e-5 noise
    np.testing.assert_allclose(G["gates"][sg][keep], R["gates"][sr][keep], rtol=0, atol=2e-4)
    # CSR offsets of the two record sets (group_records, primitive_csr.py:23-29).  The per-primitive record counts of
    # the two sets differ by at most the records that are not common to both (every record of a pixel whose count
    # differs, and both records of a position whose ids differ), and a prefix sum cannot differ by more than that.
    n = ps.n
    off_g, _ = primitive_csr.group_order(out[2], n)
    off_r, _ = primitive_csr.group_order(ref_out[2], n)
    diff = (off_g - off_r).abs().max().item()
    uncommon = int(cr[~same].sum() + cg[~same].sum() + 2 * (~ids_equal).sum())
    assert uncommon <= 4e-3 * (R["ids"].size + G["ids"].size), (uncommon, R["ids"].size)
    assert diff <= uncommon, (diff, uncommon)
    if uncommon == 0:
        assert torch.equal(off_g, off_r)
    # record totals agree to the same bound
    assert abs(int(R["ids"].size) - int(G["ids"].size)) <= uncommon
    print(f"{name}: records ref={R['ids'].size} here={G['ids'].size}, pixels with a different count: {(~same).sum()}, "
          f"positions with a different id: {(~ids_equal).sum()}, max CSR offset difference {diff}")


@pytest.mark.parametrize("name", ["tiny", "ragged", "dense"])
def test_reference_arithmetic_reproduces_reference_records_exactly(ref, name):
    """hit_arith = 1: key, hit decision and hit values in the reference kernels' own arithmetic.  Per-pixel record
    counts, record ids (hence compositing order) and the CSR offsets of render_tiles_training_records must then be
    equal, not close; the hit values (x6, decay) are the same bits."""
    from mlp_splatting_b200 import primitive_csr
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES[name])
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    P = cam["W"] * cam["H"]
    x17 = x + [torch.zeros((P, 3), device=dev), torch.zeros(P, device=dev)]
    ref_out = ref.render_tiles_training_records(x17, cam["W"], cam["H"], 8, 5e-3, 1.5, 2.0)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    out = r.render_records(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True, hit_arith=1)
    assert torch.equal(out[7], ref_out[7]), "per-pixel record offsets differ"
    assert torch.equal(out[2], ref_out[2]), "record ids differ"
    assert torch.equal(out[3], ref_out[3]), "x6 (ray direction, hit offset) differs in a bit"
    assert torch.equal(out[4][:, 6], ref_out[4][:, 6]), "decay differs in a bit"
    off_g, _ = primitive_csr.group_order(out[2], ps.n)
    off_r, _ = primitive_csr.group_order(ref_out[2], ps.n)
    assert torch.equal(off_g, off_r)
    assert (out[0] - ref_out[0]).abs().max().item() <= 1e-4


def test_feature_map_matches_reference_kernel(ref):
    """render_tiles_forward_tilecenter_with_feat (np_tile_kernels.cu:6114), slots 4, 512 channels."""
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES["ragged"])
    rng = np.random.default_rng(5)
    fa = rng.normal(0, 0.2, (scene["positions"].shape[0], 4, 512)).astype(np.float32)
    scene = dict(scene, feat_attr=fa)
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    rgb_r, alpha_r, feat_r = ref.render_tiles_forward_tilecenter_with_feat(*x, _t(fa, dev), 1.5, 2.0, cam["W"], cam["H"], 8, 8, 5e-3)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    rgb, _ = r.render(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True, want_feat=True)
    assert (rgb - rgb_r).abs().max().item() <= 1e-4
    assert (r.feat - feat_r).abs().max().item() <= 1e-4


def test_contribution_statistics_match_reference_kernel(ref):
    """render_tiles_forward_tilecenter_stats (np_tile_kernels.cu:5349-5430): the statistics kernel itself."""
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES["tiny"])
    n = scene["positions"].shape[0]
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    gt = torch.rand((cam["W"] * cam["H"], 3), device=dev, generator=torch.Generator(device=dev).manual_seed(3))
    sw, mw = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    hits = torch.zeros(n, device=dev, dtype=torch.int32)
    swe, cc = torch.zeros(n, device=dev), torch.zeros(n, device=dev, dtype=torch.int32)
    F = int(x[7].numel())
    rgb_r, alpha_r = ref.render_tiles_forward_tilecenter_stats(
        x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], x[8], F, x[9], x[10], x[11], x[12], x[13], x[14],
        int(x[9].shape[0]), int(x[9].shape[1]), int(x[9].shape[2]), cam["W"], cam["H"], 8, 8, 5e-3, gt, sw, mw, hits, swe, cc)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    s2 = (gt, torch.zeros_like(sw), torch.zeros_like(mw), torch.zeros_like(hits), torch.zeros_like(swe), torch.zeros_like(cc))
    rgb, alpha = r.render(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True, prim_stats=s2,
                          sort_key=1)   # this kernel sorts by Euclidean depth on the tile-centre ray (np_tile_kernels.cu:2248-2256)
    assert (rgb - rgb_r).abs().max().item() <= 1e-4
    assert torch.allclose(s2[1], sw, rtol=1e-4, atol=1e-4) and torch.allclose(s2[2], mw, rtol=0, atol=5e-5)
    assert torch.allclose(s2[4], swe, rtol=1e-3, atol=3e-3)
    assert (s2[3] - hits).abs().sum().item() <= max(2, int(2e-4 * hits.sum().item()))
    assert (s2[5] - cc).abs().sum().item() <= max(2, int(1e-3 * cc.sum().item()))
    assert hits.sum().item() > 1000


def test_bf16_forward_matches_reference_wmma_kernel(ref):
    """render_tiles_rgb_wmma with bf16=True (rgb_wmma.cuh:225) vs the bfloat16 operand mode of this library."""
    from mlp_splatting_b200 import _lib as L
    from mlp_splatting_b200.engine import PackedScene
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES["tiny"])
    f = oracle_frame(scene, cam, 5e-3, precision=2, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    rgb_r, alpha_r = ref.render_tiles_rgb_wmma(x, cam["W"], cam["H"], 5e-3, True)
    ps = PackedScene(scene["positions"], scene["log_scales"], scene["quats"], *[scene[k] for k in WKEYS],
                     scene["freq"], scene["att"], device=dev, pack_f16=False, pack_bf16=True)
    r = _renderer(cam, dev)
    rgb, alpha = r.render(ps, x[0], x[1], 5e-3, precision=L.PRECISION_BF16, tile_lists=(x[5], x[6]), rays_normalized=True)
    d = (rgb - rgb_r).abs()
    assert d.max().item() <= 1.5e-2 and d.mean().item() <= 3e-4, (d.max().item(), d.mean().item())
    assert (alpha - alpha_r).abs().max().item() <= 1.5e-2


@pytest.mark.parametrize("name", ["tiny", "ragged", "dense"])
def test_per_pixel_order_matches_reference_kernel(ref, name):
    """render_tiles_forward (per-pixel sort, np_tile_kernels.cu:714-926) vs sort_key = 2 of this library, FP32."""
    from mlp_splatting_b200 import _lib as L
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES[name])
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    rgb_r, alpha_r = ref.render_tiles_forward(*x, cam["W"], cam["H"], 8, 8, 5e-3)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    rgb, alpha = r.render(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True,
                          sort_key=L.ORDER_PER_PIXEL)
    d_rgb = (rgb - rgb_r).abs().max().item()
    d_a = (alpha - alpha_r).abs().max().item()
    assert d_rgb <= 1e-4 and d_a <= 1e-4, (d_rgb, d_a)


@pytest.mark.parametrize("slots,C", [(4, 96), (1, 40), (5, 33)])
def test_per_pixel_feature_map_matches_reference_kernel(ref, slots, C):
    """render_tiles_forward_per_pixel_with_feat (per-pixel sort + gated attributes) vs sort_key = 2 with a feature map."""
    from mlp_splatting_b200 import _lib as L
    dev = torch.device("cuda", 0)
    scene, cam = small_case(**CASES["ragged"])
    rng = np.random.default_rng(7 + C)
    fa = rng.normal(0, 0.2, (scene["positions"].shape[0], slots, C)).astype(np.float32)
    scene = dict(scene, feat_attr=fa if slots > 1 else fa[:, 0, :])
    f = oracle_frame(scene, cam, 5e-3, precision=0, want_masks=False)
    x = _inputs(scene, cam, f, dev)
    fa_ref = _t(fa if slots > 1 else fa[:, 0, :], dev)          # one slot is a 2-D tensor for the reference
    rgb_r, alpha_r, feat_r = ref.render_tiles_forward_per_pixel_with_feat(*x, fa_ref, 1.5, 2.0, cam["W"], cam["H"], 8, 8, 5e-3)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    rgb, alpha = r.render(ps, x[0], x[1], 5e-3, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True, want_feat=True,
                          sort_key=L.ORDER_PER_PIXEL)
    assert (rgb - rgb_r).abs().max().item() <= 1e-4 and (alpha - alpha_r).abs().max().item() <= 1e-4
    assert (r.feat - feat_r.reshape(r.feat.shape)).abs().max().item() <= 1e-4
    assert feat_r.abs().max().item() > 0.05
