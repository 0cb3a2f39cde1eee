"""Generate the golden fixtures in this directory from the reference's own Python code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/mlp-splatting

Only device-agnostic reference functions are called, on CPU:
  scannet.cumodel._encode_x6, _mlp_forward_indexed            -> mlp_eval.npz
  scannet.cumodel.IntegratedPositionalEncoding                 -> encoding.npz
  NeuralPrimitiveSceneTileCUDA.build_tilecenter_culling_from_tile_views (its device check is
  pointed at the CPU for the call; the culling code itself is untouched)  -> culling.npz
  the same method with four views and a random tile->view map                 -> mosaic.npz
  scannet.camera.ray_cone_candidates                                           -> raycone.npz
  scannet.primitive_csr.group_records, scannet.primitive_gemm.prepare_groups -> grouping.npz
  scannet.checkpoints.make_inference_checkpoint, restore_scene_state_dict,
  infer_scene_spec on a wrapped training state with prefixes, old MLP names and five feature slots
                                                                              -> checkpoint.pt
  scannet.primitive_csr.reference_weight_gradients; torch autograd through the compositing formulas
                                                                              -> backward.npz
  scannet.feature_decoder.FeatureUpsampleDecoder, scannet.eval_lseg_table2._classify_feature_map
                                                                              -> decoder.npz
The scene inputs come from this repository's seeded generator, so tests can rebuild them.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main(ref_root):
    sys.path.insert(0, ref_root)
    import scannet.cumodel as cm
    from scannet.primitive_csr import group_records
    from scannet.primitive_gemm import prepare_groups
    from mlp_splatting_b200 import synthetic as syn

    torch.manual_seed(0)
    # ---- MLP + encoding -------------------------------------------------------------------
    out = {}
    for tag, (F, H, n, R) in {"f6h32": (6, 32, 8, 256), "f1h1": (1, 1, 3, 16), "f4h16": (4, 16, 5, 64)}.items():
        sc = syn.make_scene(n, seed=100 + F, hidden=H, num_freq=F)
        rng = np.random.default_rng(7 + F)
        x6 = rng.normal(0, 0.5, (R, 6)).astype(np.float32)
        x6[:, :3] /= np.linalg.norm(x6[:, :3], axis=1, keepdims=True)
        ids = rng.integers(0, n, R).astype(np.int64)
        enc = cm._encode_x6(torch.from_numpy(x6), torch.from_numpy(sc["freq"]), torch.from_numpy(sc["att"]))
        rgb, sig = cm._mlp_forward_indexed(enc, torch.from_numpy(ids), *[torch.from_numpy(sc[k]) for k in
                                                                        ("W1", "b1", "W2", "b2", "W3", "b3")])
        out[f"{tag}_x6"], out[f"{tag}_ids"] = x6, ids.astype(np.int32)
        out[f"{tag}_enc"] = enc.numpy()
        out[f"{tag}_out"] = torch.cat([rgb, sig], 1).numpy()
        out[f"{tag}_cfg"] = np.array([F, H, n, 100 + F], np.int64)
    np.savez_compressed(os.path.join(HERE, "mlp_eval.npz"), **out)

    enc = cm.IntegratedPositionalEncoding(in_dim=6, num_frequencies=6, sigma=0.01)
    att = torch.exp(-0.5 * (enc.freq_bands ** 2) * enc.sigma2) * enc.runtime_frequency_weights
    np.savez_compressed(os.path.join(HERE, "encoding.npz"), freq=enc.freq_bands.numpy(), att=att.numpy())

    # ---- culling --------------------------------------------------------------------------
    out = {}
    for tag, (n, W, H, mu, thr, az, seed) in {
        "a": (500, 64, 48, -3.0, 5e-3, 0.0, 11), "b": (2000, 128, 96, -3.5, 5e-3, 30.0, 2026),
        "c": (300, 37, 29, -2.5, 1e-3, 200.0, 13), "d": (1500, 100, 60, -3.2, 3e-3, 90.0, 14),
    }.items():
        sc = syn.make_scene(n, seed=seed, mu=mu)
        cam = syn.make_camera(W, H, azimuth_deg=az)
        model = cm.NeuralPrimitiveSceneTileCUDA(num_primitives=n)
        with torch.no_grad():
            model.positions.copy_(torch.from_numpy(sc["positions"]))
            model.log_scales.copy_(torch.from_numpy(sc["log_scales"]))
        model.set_image_size(W, H)
        model._activate_cuda_device = lambda: torch.device("cpu")
        T = ((W + 7) // 8) * ((H + 7) // 8)
        ids, offs = model.build_tilecenter_culling_from_tile_views(
            torch.zeros(T, dtype=torch.long), torch.from_numpy(cam["view"])[None], torch.from_numpy(cam["proj"]),
            score_threshold=thr, tile_size=8)
        out[f"{tag}_cfg"] = np.array([n, W, H, seed], np.int64)
        out[f"{tag}_fcfg"] = np.array([mu, thr, az], np.float64)
        out[f"{tag}_ids"], out[f"{tag}_offsets"] = ids.numpy().astype(np.int32), offs.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "culling.npz"), **out)

    # ---- mosaic culling: every tile drawn from one of four views -----------------------------
    out = {}
    for tag, (n, W, H, mu, thr, seed) in {"m1": (2000, 128, 96, -3.5, 5e-3, 2026), "m2": (800, 67, 45, -3.0, 1e-3, 21)}.items():
        sc = syn.make_scene(n, seed=seed, mu=mu)
        cams = [syn.make_camera(W, H, azimuth_deg=90.0 * k) for k in range(4)]
        T = ((W + 7) // 8) * ((H + 7) // 8)
        tv = np.random.default_rng(seed).integers(0, 4, T).astype(np.int64)
        model = cm.NeuralPrimitiveSceneTileCUDA(num_primitives=n)
        with torch.no_grad():
            model.positions.copy_(torch.from_numpy(sc["positions"]))
            model.log_scales.copy_(torch.from_numpy(sc["log_scales"]))
        model.set_image_size(W, H)
        model._activate_cuda_device = lambda: torch.device("cpu")
        views = torch.from_numpy(np.stack([c["view"] for c in cams]))
        ids, offs = model.build_tilecenter_culling_from_tile_views(torch.from_numpy(tv), views,
                                                                   torch.from_numpy(cams[0]["proj"]),
                                                                   score_threshold=thr, tile_size=8)
        out[f"{tag}_cfg"] = np.array([n, W, H, seed], np.int64)
        out[f"{tag}_fcfg"] = np.array([mu, thr], np.float64)
        out[f"{tag}_tile_views"] = tv.astype(np.int32)
        out[f"{tag}_ids"], out[f"{tag}_offsets"] = ids.numpy().astype(np.int32), offs.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "mosaic.npz"), **out)

    # ---- ray-cone culling (scannet/camera.py:102-146) --------------------------------------
    from scannet.camera import ray_cone_candidates
    out = {}
    for tag, (n, W, H, mu, thr, az, seed) in {"r1": (2000, 128, 96, -3.5, 5e-3, 20.0, 2026),
                                              "r2": (700, 45, 38, -2.8, 1e-3, 250.0, 8)}.items():
        sc = syn.make_scene(n, seed=seed, mu=mu)
        cam = syn.make_camera(W, H, azimuth_deg=az)
        ids, offs = ray_cone_candidates(torch.from_numpy(cam["rays_o"]), torch.from_numpy(cam["rays_d"]),
                                        torch.from_numpy(sc["positions"]), torch.from_numpy(sc["log_scales"]), W, H, 8, thr)
        out[f"{tag}_cfg"] = np.array([n, W, H, seed], np.int64)
        out[f"{tag}_fcfg"] = np.array([mu, thr, az], np.float64)
        out[f"{tag}_ids"], out[f"{tag}_offsets"] = ids.numpy().astype(np.int32), offs.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "raycone.npz"), **out)

    # ---- grouping -------------------------------------------------------------------------
    counts = [0, 1, 31, 32, 33, 511, 512, 513, 1700, 0]
    ids = np.repeat(np.arange(len(counts)), counts)
    rng = np.random.default_rng(3)
    ids = ids[rng.permutation(ids.size)].astype(np.int32)
    x6 = torch.arange(ids.size * 6, dtype=torch.float32).reshape(-1, 6)
    csr = group_records(torch.from_numpy(ids), x6, x6[:, :4], len(counts))
    out = dict(ids=ids, n=np.int64(len(counts)), offsets=csr.offsets.numpy(), order=csr.record_indices.numpy())
    for seg in (512, 64):
        g = prepare_groups(csr, seg)
        out[f"seg{seg}_primitives"], out[f"seg{seg}_starts"], out[f"seg{seg}_goff"] = (
            g.primitives.numpy(), g.starts.numpy(), g.offsets.numpy())
    np.savez_compressed(os.path.join(HERE, "grouping.npz"), **out)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


def checkpoint_fixture(ref_root):
    """A small training-state checkpoint in the reference's messiest accepted form, and what the reference's
    own export / restore functions make of it."""
    sys.path.insert(0, ref_root)
    from scannet import checkpoints as ck
    from mlp_splatting_b200 import synthetic as syn
    sc = syn.make_scene(8, seed=77, hidden=32, num_freq=6, feat_dim=8, feat_slots=5)
    t = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in sc.items()}
    raw = {"module.positions": t["positions"], "module.log_scales": t["log_scales"], "module._orig_mod.quats": t["quats"],
           "module.mlps.lin1.weight": t["W1"], "module.mlps.lin1.bias": t["b1"], "module.mlps.lin2.weight": t["W2"],
           "module.mlps.lin2.bias": t["b2"], "module.mlps.lin3.weight": t["W3"], "module.mlps.lin3.bias": t["b3"],
           "module.feat_attr": t["feat_attr"], "module.encoder.freq_bands": t["freq"]}
    training = {"scene_state_dict": raw, "optimizer_state_dict": {"state": {}}, "metadata": {"iteration": 123},
                "feature_slots": 5}
    exported = ck.make_inference_checkpoint(training, storage_precision="mixed", target_feature_slots=4)
    restored = ck.restore_scene_state_dict(exported["scene_state_dict"])
    spec = ck.infer_scene_spec(exported["scene_state_dict"])
    torch.save({"training": training, "exported": exported, "restored": restored,
                "spec": {k: int(getattr(spec, k)) for k in ("num_primitives", "hidden_dim", "encoded_dim", "pe_frequencies",
                                                              "feature_dim", "feature_slots")}},
               os.path.join(HERE, "checkpoint.pt"))


DECODER_CASES = {"small": dict(in_dim=24, hidden=32, out_dim=40, classes=7, W=13, H=9, seed=41, keep=1),
                 "lseg": dict(in_dim=128, hidden=128, out_dim=512, classes=20, W=20, H=19, seed=42, keep=16)}


def decoder_fixture(ref_root):
    """decoder.npz: the reference decoder and text query on seeded weights and maps (tests rebuild the inputs from
    the same seeds); of the decoded map every keep-th channel is stored."""
    sys.path.insert(0, ref_root)
    import importlib
    from scannet.feature_decoder import FeatureUpsampleDecoder
    ev = importlib.import_module("scannet.eval_lseg_table2")
    from mlp_splatting_b200 import synthetic as syn
    out = {}
    for tag, c in DECODER_CASES.items():
        w, text = syn.make_decoder(c["in_dim"], c["hidden"], c["out_dim"], c["classes"], seed=c["seed"])
        x = syn.make_feature_map(c["W"], c["H"], c["in_dim"], seed=c["seed"] + 100)
        dec = FeatureUpsampleDecoder(c["in_dim"], c["out_dim"], c["hidden"]).eval()
        dec.load_state_dict({k: torch.from_numpy(v) for k, v in w.items()})
        with torch.no_grad():
            y = dec(torch.from_numpy(x).permute(2, 0, 1).unsqueeze(0).float()).squeeze(0).permute(1, 2, 0).contiguous()
            lab = ev._classify_feature_map(y, torch.from_numpy(text))
        out[f"{tag}_decoded"] = y.numpy()[..., ::c["keep"]].copy()
        out[f"{tag}_labels"] = lab.numpy().astype(np.int64)
    np.savez_compressed(os.path.join(HERE, "decoder.npz"), **out)


def backward_fixtures(ref_root):
    """backward.npz: (1) per-primitive weight gradients from the reference's own PyTorch statement
    (scannet.primitive_csr.reference_weight_gradients) on the record counts its test uses
    (tests/test_primitive_csr.py:91-134); (2) reverse compositing adjoints by torch autograd through the
    compositing and decay formulas (np_tile_kernels.cu:659-711, 2025-2136), the independent check of
    primitive_records_reverse."""
    sys.path.insert(0, ref_root)
    from scannet.primitive_csr import PrimitiveCSR, reference_weight_gradients
    from scannet.cumodel import _encode_x6
    out = {}
    g = torch.Generator().manual_seed(92)
    counts = torch.tensor([0, 1, 31, 32, 33, 511, 512, 513, 1700, 0])
    ids = torch.repeat_interleave(torch.arange(10, dtype=torch.int32), counts)
    R = int(ids.numel())
    x6 = torch.randn((R, 6), generator=g) * .2
    d3 = torch.randn((R, 4), generator=g)
    freq = 2. ** torch.arange(6, dtype=torch.float32)
    att = torch.exp(-.5 * freq.square() * 1.e-4)
    weights = [torch.randn((10, *shape), generator=g) * .1 for shape in [(32, 72), (32,), (32, 32), (32,), (4, 32), (4,)]]
    offsets = torch.cat((counts.new_zeros(1), counts.cumsum(0))).to(torch.int64)
    masks = torch.zeros((R, 2), dtype=torch.int32)
    bit = 1 << torch.arange(32, dtype=torch.int64)
    for p in range(10):
        b, e = int(offsets[p]), int(offsets[p + 1])
        if b == e:
            continue
        enc = _encode_x6(x6[b:e], freq, att)
        h1 = torch.relu(enc @ weights[0][p].T + weights[1][p])
        h2 = torch.relu(h1 @ weights[2][p].T + weights[3][p])
        masks[b:e, 0] = ((h1 > 0) * bit).sum(1).to(torch.int32)
        masks[b:e, 1] = ((h2 > 0) * bit).sum(1).to(torch.int32)
    csr = PrimitiveCSR(offsets, torch.arange(R), x6, d3, masks)
    expected = reference_weight_gradients(csr, freq, att, weights)
    out.update(vjp_offsets=offsets.numpy(), vjp_x6=x6.numpy(), vjp_d3=d3.numpy(), vjp_masks=masks.numpy(),
               vjp_freq=freq.numpy(), vjp_att=att.numpy())
    for k, w, e in zip(("W1", "b1", "W2", "b2", "W3", "b3"), weights, expected):
        out["vjp_" + k] = w.numpy()
        out["vjp_g" + k] = e.numpy()

    # ---- reverse compositing by autograd ----
    g = torch.Generator().manual_seed(5)
    n, pixels = 6, 40
    per_px = torch.randint(0, 7, (pixels,), generator=g)
    per_px[3] = 0
    offs = torch.cat((per_px.new_zeros(1), per_px.cumsum(0))).to(torch.int64)
    R = int(offs[-1])
    rid = torch.randint(0, n, (R,), generator=g).to(torch.int32)
    logit = (torch.randn((R, 4), generator=g)).double().requires_grad_(True)
    dvec = (torch.randn((R, 3), generator=g) * .05).double().requires_grad_(True)
    ls = (torch.randn((n, 3), generator=g) * .3 - 3.0).double().requires_grad_(True)
    qt = torch.randn((n, 4), generator=g).double()
    qt = (qt / qt.norm(dim=1, keepdim=True)).requires_grad_(True)
    grgb = torch.randn((pixels, 3), generator=g).double()
    gt = torch.randn((pixels,), generator=g).double()
    w_, x_, y_, z_ = qt[rid.long()].unbind(1)
    Rm = torch.stack([1 - 2 * (y_ * y_ + z_ * z_), 2 * (x_ * y_ - w_ * z_), 2 * (x_ * z_ + w_ * y_),
                      2 * (x_ * y_ + w_ * z_), 1 - 2 * (x_ * x_ + z_ * z_), 2 * (y_ * z_ - w_ * x_),
                      2 * (x_ * z_ - w_ * y_), 2 * (y_ * z_ + w_ * x_), 1 - 2 * (x_ * x_ + y_ * y_)], 1).view(R, 3, 3)
    qloc = torch.einsum("rij,ri->rj", Rm, dvec)                       # R^T d
    m = torch.exp(-2 * ls[rid.long()])
    decay = torch.exp(-0.5 * (qloc * qloc * m).sum(1))
    rgbv = torch.sigmoid(logit[:, :3])
    sraw = torch.nn.functional.softplus(logit[:, 3])
    alpha = 1 - torch.exp(-sraw * decay)
    loss = 0.
    trans_before = torch.zeros(R, dtype=torch.double)
    for px in range(pixels):
        T = torch.ones((), dtype=torch.double)
        C = torch.zeros(3, dtype=torch.double)
        for r in range(int(offs[px]), int(offs[px + 1])):
            trans_before[r] = T.detach()
            C = C + T * alpha[r] * rgbv[r]
            T = T * (1 - alpha[r])
        loss = loss + (grgb[px] * C).sum() + gt[px] * T
    loss.backward()
    gp = torch.zeros((n, 3), dtype=torch.double).index_add_(0, rid.long(), dvec.grad)
    raw = torch.stack([rgbv[:, 0], rgbv[:, 1], rgbv[:, 2], sraw, trans_before, alpha, decay, logit[:, 3]], 1).detach()
    x6r = torch.cat([torch.zeros((R, 3), dtype=torch.double), dvec.detach()], 1)
    out.update(rev_ids=rid.numpy(), rev_offsets=offs.numpy(), rev_x6=x6r.float().numpy(), rev_raw=raw.float().numpy(),
               rev_logs=ls.detach().float().numpy(), rev_quats=qt.detach().float().numpy(),
               rev_grgb=grgb.float().numpy(), rev_gt=gt.float().numpy(), rev_d4=logit.grad.float().numpy(),
               rev_gp=gp.float().numpy(), rev_gs=ls.grad.float().numpy(), rev_gq=qt.grad.float().numpy())
    np.savez_compressed(os.path.join(HERE, "backward.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/mlp-splatting [fixture ...]")
    root = sys.argv[1]
    makers = {"main": main, "checkpoint": checkpoint_fixture, "backward": backward_fixtures, "decoder": decoder_fixture}
    for name in (sys.argv[2:] or list(makers)):
        makers[name](root)
