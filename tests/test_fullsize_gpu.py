"""Full-size checks on the bench workload (100,000 primitives, 1200x680): properties that need no CPU render,
and the reference's own CUDA kernels as the yardstick where they have been built (oracle/build_ref.py)."""
import numpy as np
import pytest
import torch

from tests.helpers import WKEYS

pytestmark = pytest.mark.gpu
THR = 5e-3


@pytest.fixture(scope="module")
def world():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mlp_splatting_b200 import synthetic as syn
    from mlp_splatting_b200.engine import FrameRenderer, PackedScene, normalize_rows
    dev = torch.device("cuda", 0)
    scene, cams, cfg = syn.make_workload("single_100k_1200x680")
    cam = cams[0]
    ps = PackedScene(scene["positions"], scene["log_scales"], scene["quats"], *[scene[k] for k in WKEYS],
                     scene["freq"], scene["att"], device=dev, pack_f16=True)
    r = FrameRenderer(cam["W"], cam["H"], device=dev)
    ro, rd = torch.from_numpy(cam["rays_o"]).to(dev), torch.from_numpy(cam["rays_d"]).to(dev)
    return dict(dev=dev, scene=scene, cam=cam, ps=ps, r=r, ro=ro, rd=rd, rdu=normalize_rows(rd))


def _render(w, **kw):
    rgb, a = w["r"].render(w["ps"], w["ro"], w["rd"], THR, view=w["cam"]["view"], proj=w["cam"]["proj"], **kw)
    return rgb.clone(), a.clone(), w["r"].last_stats


def test_image_is_independent_of_pretest_and_schedule(world):
    from mlp_splatting_b200 import _lib as L
    base = _render(world, precision=L.PRECISION_F16)
    for kw in (dict(tile_pretest=False), dict(waves=[64, 2048]), dict(waves=[16, 16, 32, 64, 128, 256, 2048]),
               dict(waves=[48, 48, 2048], tile_pretest=False)):
        rgb, a, st = _render(world, precision=L.PRECISION_F16, **kw)
        assert torch.equal(rgb, base[0]) and torch.equal(a, base[1]), kw
        assert st.used == base[2].used and st.pairs == base[2].pairs
    st = base[2]
    assert 0 < st.pairs_kept < st.pairs and st.used <= st.records
    assert st.max_tile_len <= 1536
    # fp16 tensor-core frame against the FP32 frame: the tolerance the path is specified to
    rgb32, a32, _ = _render(world, precision=L.PRECISION_F32)
    assert (rgb32 - base[0]).abs().max().item() <= 2e-3 and (a32 - base[1]).abs().max().item() <= 2e-3


def test_pretest_keeps_every_pair_with_a_hit(world):
    """At full size: every (tile, primitive) pair whose geometric hit mask is not empty survives the pre-test."""
    r, ps = world["r"], world["ps"]
    prims, offs = r.bin(ps, world["cam"]["view"], world["cam"]["proj"], THR)
    M = int(prims.numel())
    full = r.sort(ps, world["ro"], world["rdu"], M).clone()
    geo = r.hit_masks(ps, world["ro"], world["rdu"], THR, M).clone()
    offs = offs.clone()
    _render(world)                                   # leaves the kept lists (+ -1 padding) in sorted_prims
    kept = r.sorted_prims[:M].clone()
    T = offs.numel() - 1
    tile_of = torch.repeat_interleave(torch.arange(T, device=offs.device), (offs[1:] - offs[:-1]).long())
    n = ps.n
    key_full = tile_of.long() * n + full.long()
    valid = kept >= 0
    key_kept = tile_of.long()[valid] * n + kept.long()[valid]
    hit_keys = key_full[geo != 0]
    assert torch.isin(hit_keys, key_kept).all()
    assert int(valid.sum()) == r.last_stats.pairs_kept
    # and it is tight: few kept pairs without any hit
    assert int(valid.sum()) <= 1.05 * int((geo != 0).sum())


def test_fp16_frame_matches_reference_wmma_kernel_at_full_size(world):
    """The reference's render_tiles_rgb_wmma (rgb_wmma.cuh:225) on the same 100k scene and the same tile lists."""
    from oracle import build_ref
    ref = build_ref.load_module()
    if ref is None:
        pytest.skip("reference extension not built (python oracle/build_ref.py)")
    from mlp_splatting_b200.engine import normalize_rows
    r, ps, sc, dev = world["r"], world["ps"], world["scene"], world["dev"]
    prims, offs = r.bin(ps, world["cam"]["view"], world["cam"]["proj"], THR)
    prims, offs = prims.clone(), offs.clone()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    x = [world["ro"], world["rdu"], t(sc["positions"]), t(sc["log_scales"]), normalize_rows(t(sc["quats"])), prims, offs,
         t(sc["freq"]), t(sc["att"])] + [t(sc[k]) for k in WKEYS]
    rgb_r, alpha_r = ref.render_tiles_rgb_wmma(x, world["cam"]["W"], world["cam"]["H"], THR, False)
    rgb, alpha, _ = _render(world)
    # 2e-3 is the tolerance the path is specified to.  Among the 45 million (pixel, primitive) hit tests of this
    # frame a handful sit within 1e-6 relative of the threshold, where the reference's hardware exp and this
    # library's IEEE-only exp may decide differently; such a pixel gains or loses one faint record.  So: all but
    # at most ten pixels within 2e-3, none further than 2e-2, and a mean error far below either.
    err = torch.maximum((rgb - rgb_r).abs().max(dim=1).values, (alpha - alpha_r).abs()[:, 0])
    assert int((err > 2e-3).sum()) <= 10, int((err > 2e-3).sum())
    assert err.max().item() <= 2e-2
    assert (rgb - rgb_r).abs().mean().item() <= 5e-5
    assert alpha_r.mean().item() > 0.2          # the frame is not empty


def test_per_pixel_order_matches_reference_kernel_at_full_size(world):
    """The reference's render_tiles_forward (per-pixel sort, np_tile_kernels.cu:714-926) on the 100k scene: either
    both refuse (a pixel with more than 256 hits) or the FP32 images agree."""
    from oracle import build_ref
    ref = build_ref.load_module()
    if ref is None:
        pytest.skip("reference extension not built (python oracle/build_ref.py)")
    from mlp_splatting_b200 import _lib as L
    from mlp_splatting_b200.engine import RenderError, normalize_rows
    r, ps, sc, dev = world["r"], world["ps"], world["scene"], world["dev"]
    prims, offs = r.bin(ps, world["cam"]["view"], world["cam"]["proj"], THR)
    prims, offs = prims.clone(), offs.clone()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    x = [world["ro"], world["rdu"], t(sc["positions"]), t(sc["log_scales"]), normalize_rows(t(sc["quats"])), prims, offs,
         t(sc["freq"]), t(sc["att"])] + [t(sc[k]) for k in WKEYS]
    try:
        rgb_r, alpha_r = ref.render_tiles_forward(*x, world["cam"]["W"], world["cam"]["H"], 8, 8, THR)
    except RuntimeError as e:
        assert "per-pixel intersection capacity 256 exceeded" in str(e)
        with pytest.raises(RenderError, match="per-pixel intersection capacity 256 exceeded"):
            _render(world, precision=L.PRECISION_F32, sort_key=L.ORDER_PER_PIXEL)
        return
    rgb, alpha, st = _render(world, precision=L.PRECISION_F32, sort_key=L.ORDER_PER_PIXEL)
    assert st.waves == 1 and st.records > st.used > 0
    err = torch.maximum((rgb - rgb_r).abs().max(dim=1).values, (alpha - alpha_r).abs()[:, 0])
    assert int((err > 1e-4).sum()) <= 10, int((err > 1e-4).sum())
    assert err.max().item() <= 2e-2
    # and the order matters at this size too
    rgb_t, _a, _s = _render(world, precision=L.PRECISION_F32)
    assert (rgb_t - rgb).abs().max().item() > 0.05
