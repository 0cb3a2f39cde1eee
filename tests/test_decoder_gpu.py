"""Feature decoder and text query on the GPU against the CPU restatement and tests/golden/decoder.npz (outputs of the
reference's FeatureUpsampleDecoder and _classify_feature_map, scannet/feature_decoder.py:5-19 and
scannet/eval_lseg_table2.py:622-641).

Tolerances.  The tensor-core decoder rounds inputs, weights and hidden activations to binary16 and accumulates in
FP32, like the tensor-core MLP: against the restatement with the same rounding model the decoded map agrees to
2e-3 absolute (summation order, rare one-ulp flips of a hidden activation), against the FP32 reference to 1e-2.
Labels are compared where the winner is clear: a pixel may differ only if its best and second-best cosine logits
are closer than the stated margin."""
import os

import numpy as np
import pytest
import torch

from mlp_splatting_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
CASES = {"small": dict(in_dim=24, hidden=32, out_dim=40, classes=7, W=13, H=9, seed=41, keep=1),
         "lseg": dict(in_dim=128, hidden=128, out_dim=512, classes=20, W=20, H=19, seed=42, keep=16)}


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def _decoder(c, dev):
    from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder
    w, text = syn.make_decoder(c["in_dim"], c["hidden"], c["out_dim"], c.get("classes", 0), seed=c["seed"])
    dec = FeatureUpsampleDecoder(c["in_dim"], c["out_dim"], c["hidden"], device=dev)
    dec.load_state_dict({k: torch.from_numpy(v) for k, v in w.items()})
    x = syn.make_feature_map(c["W"], c["H"], c["in_dim"], seed=c["seed"] + 100)
    return dec, w, text, x


@pytest.mark.parametrize("tag", list(CASES))
def test_decoded_map_matches_oracle_and_reference(dev, tag):
    from oracle import oracle as orc
    fx = np.load(os.path.join(HERE, "golden", "decoder.npz"))
    c = CASES[tag]
    dec, w, text, x = _decoder(c, dev)
    got = dec.decode_hwc(torch.from_numpy(x).to(dev)).cpu().numpy()
    want16 = orc.decode_features(x, w, precision=1)
    assert np.abs(got - want16).max() <= 2e-3
    assert np.abs(got[..., ::c["keep"]] - fx[f"{tag}_decoded"]).max() <= 1e-2
    # the module-style call is the same map in NCHW
    nchw = dec(torch.from_numpy(x).to(dev).permute(2, 0, 1).unsqueeze(0))
    assert nchw.shape == (1, c["out_dim"], c["H"], c["W"])
    assert torch.equal(nchw[0].permute(1, 2, 0).cpu(), torch.from_numpy(got))


@pytest.mark.parametrize("tag", list(CASES))
def test_fused_query_matches_oracle_and_reference(dev, tag):
    from oracle import oracle as orc
    fx = np.load(os.path.join(HERE, "golden", "decoder.npz"))
    c = CASES[tag]
    dec, w, text, x = _decoder(c, dev)
    t = torch.from_numpy(text).to(dev)
    got = dec.classify(torch.from_numpy(x).to(dev), t).cpu().numpy()
    assert got.dtype == np.int64 and got.shape == (c["H"], c["W"])
    labels16, margin16 = orc.classify_features(orc.decode_features(x, w, precision=1), text)
    differ = got != labels16
    assert not differ[margin16 > 2e-3].any(), (int(differ.sum()), float(margin16[differ].max()))
    labels32, margin32 = orc.classify_features(orc.decode_features(x, w), text)
    assert np.array_equal(labels32, fx[f"{tag}_labels"])
    differ = got != fx[f"{tag}_labels"]
    assert not differ[margin32 > 5e-3].any() and differ.mean() <= 0.05
    # a second call reuses the packed image and gives the same labels
    assert np.array_equal(dec.classify(torch.from_numpy(x).to(dev), t).cpu().numpy(), got)


@pytest.mark.parametrize("W,H", [(1, 1), (8, 16), (9, 17), (7, 40), (203, 131)])
def test_image_edges_and_many_tiles(dev, W, H):
    """Images smaller than a tile, exactly one tile, one pixel over, and more tiles than SMs (every CTA walks
    several tiles and the weight ring wraps many times)."""
    from oracle import oracle as orc
    c = dict(in_dim=16, hidden=32, out_dim=64, classes=11, W=W, H=H, seed=50 + W)
    dec, w, text, x = _decoder(c, dev)
    got = dec.decode_hwc(torch.from_numpy(x).to(dev)).cpu().numpy()
    want = orc.decode_features(x, w, precision=1)
    assert np.abs(got - want).max() <= 2e-3
    lab = dec.classify(torch.from_numpy(x).to(dev), torch.from_numpy(text).to(dev)).cpu().numpy()
    l16, m16 = orc.classify_features(want, text)
    assert not (lab != l16)[m16 > 2e-3].any()


def test_hidden_64_and_odd_widths(dev):
    from oracle import oracle as orc
    c = dict(in_dim=21, hidden=64, out_dim=130, classes=3, W=30, H=21, seed=77)
    dec, w, text, x = _decoder(c, dev)
    got = dec.decode_hwc(torch.from_numpy(x).to(dev)).cpu().numpy()
    assert np.abs(got - orc.decode_features(x, w, precision=1)).max() <= 2e-3


def test_out_of_range_input_is_reported(dev):
    c = CASES["small"]
    dec, w, text, x = _decoder(c, dev)
    x = x.copy()
    x[3, 4, 5] = 1.0e6
    with pytest.raises(FloatingPointError):
        dec.decode_hwc(torch.from_numpy(x).to(dev))
    # the status was cleared: the next call works
    x[3, 4, 5] = 0.0
    dec.decode_hwc(torch.from_numpy(x).to(dev))


def test_limits_are_rejected(dev):
    from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder
    w, _ = syn.make_decoder(8, 48, 16, seed=1)
    dec = FeatureUpsampleDecoder(8, 16, 48, device=dev).load_state_dict({k: torch.from_numpy(v) for k, v in w.items()})
    with pytest.raises(ValueError, match="limits"):
        dec.decode_hwc(torch.zeros(4, 4, 8, device=dev))


@pytest.mark.parametrize("D,C,P", [(512, 20, (37, 53)), (40, 7, (9, 13)), (600, 150, (16, 16)), (3, 1, (5, 5))])
def test_full_width_query_matches_oracle(dev, D, C, P):
    from mlp_splatting_b200.feature_decoder import classify_feature_map
    from oracle import oracle as orc
    rng = np.random.default_rng(D + C)
    feat = rng.normal(size=(*P, D)).astype(np.float32)
    feat[0, 0] = 0.0                                   # an all-zero row takes label 0
    text = rng.normal(size=(C, D)).astype(np.float32)
    got = classify_feature_map(torch.from_numpy(feat).to(dev), torch.from_numpy(text).to(dev)).cpu().numpy()
    want, margin = orc.classify_features(feat, text)
    assert got.shape == P and got.dtype == np.int64 and got[0, 0] == 0
    assert not (got != want)[margin > 1e-5].any()


def test_text_query_view_of_a_scene_gives_the_full_width_labels(dev):
    """Rendering class scores from PackedScene.with_text_query() and taking the arg-max equals querying the
    full-width rendered feature map (compositing is linear in the features)."""
    from mlp_splatting_b200.feature_decoder import classify_feature_map, score_labels
    from oracle import oracle as orc
    from test_parity_gpu import CASES as SCENES, _packed, _renderer, _t, small_case
    scene, cam = small_case(**SCENES["ragged"])
    rng = np.random.default_rng(9)
    D, C = 64, 6
    scene = dict(scene, feat_attr=rng.normal(0, 0.2, (scene["positions"].shape[0], 4, D)).astype(np.float32))
    text = rng.normal(size=(C, D)).astype(np.float32)
    ps, r = _packed(scene, dev), _renderer(cam, dev)
    args = (_t(cam["rays_o"], dev), _t(cam["rays_d"], dev), 5e-3)
    r.render(ps, *args, view=cam["view"], proj=cam["proj"], precision=0, want_feat=True)
    full = r.feat.view(cam["H"], cam["W"], D).clone()
    want = classify_feature_map(full, torch.from_numpy(text).to(dev)).cpu().numpy()
    view = ps.with_text_query(torch.from_numpy(text))
    assert view.feat_dim == C and view.geom is ps.geom and view.w16 is ps.w16
    r.render(view, *args, view=cam["view"], proj=cam["proj"], precision=0, want_feat=True)
    scores = r.feat.view(cam["H"], cam["W"], C).clone()
    got = score_labels(scores).cpu().numpy()
    _labels, margin = orc.classify_features(full.cpu().numpy(), text)
    differ = got != want
    assert not differ[margin > 1e-4].any() and differ.mean() < 0.01
    # pixels nothing covers have an all-zero feature row and take label 0 on both routes
    empty = (full.abs().sum(2) == 0).cpu().numpy()
    assert empty.any() and (got[empty] == 0).all() and (want[empty] == 0).all()
    with pytest.raises(ValueError, match="Feature dim mismatch"):
        ps.with_text_query(torch.zeros(3, D + 1))


def test_full_size_fused_query_agrees_with_decode_then_query(dev):
    """At 1200x680 with the 128-128-512 decoder: the fused kernel (text product folded into the last layer) and the
    two-step route (decoded 512-channel map, then the FP32 full-width query) must label the pixels alike -- they
    differ only by the binary16 rounding of the folded matrix -- and both must be deterministic."""
    from mlp_splatting_b200.feature_decoder import classify_feature_map
    c = dict(in_dim=128, hidden=128, out_dim=512, classes=20, W=1200, H=680, seed=61)
    dec, w, text, x = _decoder(c, dev)
    xt, t = torch.from_numpy(x).to(dev), torch.from_numpy(text).to(dev)
    fused = dec.classify(xt, t)
    two_step = classify_feature_map(dec.decode_hwc(xt), t)
    assert fused.shape == (680, 1200) and fused.dtype == torch.int64
    agree = (fused == two_step).float().mean().item()
    assert agree >= 0.995, agree
    assert torch.equal(fused, dec.classify(xt, t))
    counts = torch.bincount(fused.reshape(-1), minlength=20)
    assert int((counts > 0).sum()) >= 10            # a real segmentation, not one label
