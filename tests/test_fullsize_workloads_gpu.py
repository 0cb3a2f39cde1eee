"""Full-size parity of the other named workloads: the reference's own CUDA kernels (oracle/build_ref.py) on the same
device tensors and tile lists where a reference implementation exists, the CPU restatement on a band of tile rows
where none does (64-wide hidden layers).  Also the record / CSR comparison of the 100,000-primitive bench frame with
the reference's record kernel, so that the number of threshold flips at full size is an asserted figure.
"""
import numpy as np
import pytest
import torch

from tests.helpers import WKEYS

pytestmark = pytest.mark.gpu
THR = 5e-3


def _setup(name, want_feat=False, pack_f16=True):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mlp_splatting_b200 import synthetic as syn
    from mlp_splatting_b200.engine import FrameRenderer, PackedScene, normalize_rows
    dev = torch.device("cuda", 0)
    scene, cams, cfg = syn.make_workload(name)
    ps = PackedScene(scene["positions"], scene["log_scales"], scene["quats"], *[scene[k] for k in WKEYS],
                     scene["freq"], scene["att"], feat_attr=scene.get("feat_attr") if want_feat else None,
                     device=dev, pack_f16=pack_f16)
    return dict(dev=dev, scene=scene, cams=cams, cfg=cfg, ps=ps, normalize_rows=normalize_rows, FrameRenderer=FrameRenderer)


def _ref_module():
    from oracle import build_ref
    ref = build_ref.load_module()
    if ref is None:
        pytest.skip("reference extension not built (python oracle/build_ref.py)")
    return ref


def _ref_inputs(w, cam, r):
    """The reference entry points' 15 tensors, with this library's own (bit-exact) tile lists."""
    dev, sc, ps = w["dev"], w["scene"], w["ps"]
    ro, rd = torch.from_numpy(cam["rays_o"]).to(dev), torch.from_numpy(cam["rays_d"]).to(dev)
    rdu = w["normalize_rows"](rd)
    prims, offs = r.bin(ps, cam["view"], cam["proj"], THR)
    prims, offs = prims.clone(), offs.clone()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    x = [ro, rdu, ps.positions, ps.log_scales, ps.quats_unit, prims, offs, ps.freq, ps.att] + [getattr(ps, k) for k in WKEYS]
    return x, ro, rdu


def _pixel_error(*pairs):
    err = None
    for a, b in pairs:
        e = (a - b).abs().reshape(a.shape[0], -1).max(dim=1).values
        err = e if err is None else torch.maximum(err, e)
    return err


def test_reference_arithmetic_gives_the_reference_record_sets_at_full_size():
    """hit_arith = 1 on the 100,000-primitive frame: record counts per pixel, record ids and CSR offsets equal those of
    render_tiles_training_records, exactly."""
    from mlp_splatting_b200 import primitive_csr
    ref = _ref_module()
    w = _setup("single_100k_1200x680", pack_f16=False)
    cam = w["cams"][0]
    r = w["FrameRenderer"](cam["W"], cam["H"], device=w["dev"])
    x, ro, rdu = _ref_inputs(w, cam, r)
    P = cam["W"] * cam["H"]
    x17 = x + [torch.zeros((P, 3), device=w["dev"]), torch.zeros(P, device=w["dev"])]
    ref_out = ref.render_tiles_training_records(x17, cam["W"], cam["H"], 8, THR, 1.5, 2.0)
    ids_r, off_r = ref_out[2], ref_out[7]
    del ref_out
    out = r.render_records(w["ps"], ro, rdu, THR, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True, hit_arith=1)
    n_px = int((out[7] != off_r).sum())
    n_id = int((out[2] != ids_r).sum()) if out[2].numel() == ids_r.numel() else -1
    print(f"bench frame, reference arithmetic: records ref={ids_r.numel()} here={out[2].numel()}; offsets that differ {n_px}; ids that differ {n_id}")
    assert n_px == 0 and n_id == 0
    csr_g, _ = primitive_csr.group_order(out[2], w["ps"].n)
    csr_r, _ = primitive_csr.group_order(ids_r, w["ps"].n)
    assert torch.equal(csr_g, csr_r)


def test_records_and_csr_of_the_bench_frame_match_reference_kernel():
    """render_tiles_training_records (np_tile_kernels.cu:6994) on the 100,000-primitive frame, FP32: per-pixel record
    lists, ids and CSR offsets, with the differences (threshold flips of the kind the arithmetic contract predicts)
    counted and bounded."""
    from mlp_splatting_b200 import primitive_csr
    ref = _ref_module()
    w = _setup("single_100k_1200x680", pack_f16=False)
    cam = w["cams"][0]
    r = w["FrameRenderer"](cam["W"], cam["H"], device=w["dev"])
    x, ro, rdu = _ref_inputs(w, cam, r)
    P = cam["W"] * cam["H"]
    x17 = x + [torch.zeros((P, 3), device=w["dev"]), torch.zeros(P, device=w["dev"])]
    ref_out = ref.render_tiles_training_records(x17, cam["W"], cam["H"], 8, THR, 1.5, 2.0)
    ids_r, off_r = ref_out[2], ref_out[7]
    del ref_out
    out = r.render_records(w["ps"], ro, rdu, THR, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True)
    ids_g, off_g = out[2], out[7]
    cr, cg = off_r[1:] - off_r[:-1], off_g[1:] - off_g[:-1]
    same = cr == cg
    n_px = int((~same).sum())
    assert n_px <= 40, f"{n_px} of {P} pixels differ in record count"
    pr = torch.repeat_interleave(torch.arange(P, device=w["dev"]), cr)
    pg = torch.repeat_interleave(torch.arange(P, device=w["dev"]), cg)
    ids_equal = ids_r[same[pr]] == ids_g[same[pg]]
    n_id = int((~ids_equal).sum())
    # two candidates of a tile whose sort keys agree to the last bits may swap (this library's keys use the IEEE-only
    # exponential, the reference's the hardware one): every pixel of the tile that composites both then shows two ids
    assert n_id <= 1000, f"{n_id} record ids differ on pixels with equal counts"
    uncommon = int(cr[~same].sum() + cg[~same].sum()) + 2 * n_id
    csr_g, _ = primitive_csr.group_order(ids_g, w["ps"].n)
    csr_r, _ = primitive_csr.group_order(ids_r, w["ps"].n)
    diff = int((csr_g - csr_r).abs().max())
    assert diff <= uncommon
    assert abs(int(ids_r.numel()) - int(ids_g.numel())) <= uncommon
    assert int(ids_r.numel()) > 5_000_000
    print(f"bench frame: records ref={ids_r.numel()} here={ids_g.numel()}; pixels with a different count {n_px}; "
          f"differing ids {n_id}; max CSR offset difference {diff}")


def test_feature_frame_matches_reference_kernel_at_full_size():
    """render_tiles_forward_tilecenter_with_feat (np_tile_kernels.cu:6114) on the 250,000-primitive feature workload:
    rgb, alpha and the 512-channel feature map, FP32."""
    ref = _ref_module()
    w = _setup("feature_250k_1200x680", want_feat=True, pack_f16=False)
    cam = w["cams"][0]
    r = w["FrameRenderer"](cam["W"], cam["H"], device=w["dev"])
    x, ro, rdu = _ref_inputs(w, cam, r)
    rgb_r, alpha_r, feat_r = ref.render_tiles_forward_tilecenter_with_feat(*x, w["ps"].feat_attr, 1.5, 2.0, cam["W"], cam["H"], 8, 8, THR)
    rgb, alpha = r.render(w["ps"], ro, rdu, THR, precision=0, tile_lists=(x[5], x[6]), rays_normalized=True, want_feat=True)
    err = _pixel_error((rgb, rgb_r), (alpha, alpha_r))
    ferr = _pixel_error((r.feat, feat_r.reshape(r.feat.shape)))
    figures = dict(rgb_over_1e4=int((err > 1e-4).sum()), rgb_over_1e3=int((err > 1e-3).sum()), rgb_max=err.max().item(),
                   feat_over_1e3=int((ferr > 1e-3).sum()), feat_max=ferr.max().item(), feat_mean=ferr.mean().item())
    print("feature frame vs reference kernel:", figures)
    # FP32 on both sides, hardware sin / cos / exp on both sides: the images agree to 1e-4 except where a hit decision
    # or a sort order flipped (a pixel then gains, loses or reorders one faint record)
    assert figures["rgb_over_1e4"] <= 200 and figures["rgb_over_1e3"] <= 20 and figures["rgb_max"] <= 2e-2, figures
    assert figures["feat_over_1e3"] <= 60 and figures["feat_max"] <= 0.05 and figures["feat_mean"] <= 5e-6, figures
    assert feat_r.abs().max().item() > 0.1 and alpha_r.mean().item() > 0.2


def test_fourview_frame_matches_reference_wmma_kernel():
    """render_tiles_rgb_wmma (rgb_wmma.cuh:225) on one view of the 500,000-primitive four-view workload, fp16."""
    ref = _ref_module()
    w = _setup("fourview_500k_1200x680")
    cam = w["cams"][1]
    r = w["FrameRenderer"](cam["W"], cam["H"], device=w["dev"])
    x, ro, rdu = _ref_inputs(w, cam, r)
    rgb_r, alpha_r = ref.render_tiles_rgb_wmma(x, cam["W"], cam["H"], THR, False)
    rgb, alpha = r.render(w["ps"], ro, rdu, THR, view=cam["view"], proj=cam["proj"], rays_normalized=True)
    err = _pixel_error((rgb, rgb_r), (alpha, alpha_r))
    assert int((err > 2e-3).sum()) <= 10, int((err > 2e-3).sum())
    assert err.max().item() <= 2e-2 and (rgb - rgb_r).abs().mean().item() <= 5e-5
    assert r.f32_fallbacks == 0 and alpha_r.mean().item() > 0.2


def test_hidden64_frame_matches_oracle_band():
    """The 72-64-64-4 network (no reference implementation: the reference stops at 32 hidden units, so parity is
    unpinned): the tensor-core frame against the CPU restatement's fp16 operand model on a band of tile rows."""
    from oracle import oracle as orc
    w = _setup("hidden64_250k_1200x680")
    assert w["ps"].hidden == 64 and w["ps"].has_f16
    cam, sc = w["cams"][0], w["scene"]
    W, H = cam["W"], cam["H"]
    r = w["FrameRenderer"](W, H, device=w["dev"])
    ro, rd = torch.from_numpy(cam["rays_o"]).to(w["dev"]), torch.from_numpy(cam["rays_d"]).to(w["dev"])
    rgb, alpha = r.render(w["ps"], ro, rd, THR, view=cam["view"], proj=cam["proj"])
    assert r.f32_fallbacks == 0
    q, rdu = orc.normalize_rows(sc["quats"]), orc.normalize_rows(cam["rays_d"])
    geom = orc.pack_geometry(sc["positions"], sc["log_scales"], q)
    prims, off = orc.bin_tiles(geom, cam["view"], cam["proj"], W, H, 8, THR)
    assert np.array_equal(r.tile_offsets.cpu().numpy(), off)
    sp = orc.sort_tiles(cam["rays_o"], rdu, geom, off, prims, W, H, 8)
    ntx, row0, rows = (W + 7) // 8, 40, 3
    res = orc.render(cam["rays_o"], rdu, geom, off, sp, W, H, 8, THR, [sc[k] for k in WKEYS], sc["freq"], sc["att"],
                     precision=1, want_masks=False, tile_range=(row0 * ntx, (row0 + rows) * ntx))
    band = slice(row0 * 8 * W, (row0 + rows) * 8 * W)
    d_rgb = np.abs(rgb.cpu().numpy()[band] - res.rgb[band]).max(axis=1)
    d_a = np.abs(alpha.cpu().numpy()[band, 0] - res.alpha[band])
    err = np.maximum(d_rgb, d_a)
    assert (err > 1e-3).sum() <= 3 and err.max() <= 2e-2, (int((err > 1e-3).sum()), float(err.max()))
    assert res.alpha[band].mean() > 0.2
