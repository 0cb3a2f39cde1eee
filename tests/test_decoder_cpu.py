"""Feature decoder and text query: the CPU restatement against tests/golden/decoder.npz, which holds the outputs of
the reference's own FeatureUpsampleDecoder (scannet/feature_decoder.py:5-19) and _classify_feature_map
(scannet/eval_lseg_table2.py:622-641) on seeded weights and maps (tests/golden/make_golden.py), and the host-side
argument checks of the product's mirror, which need no device."""
import os

import numpy as np
import pytest
import torch

from mlp_splatting_b200 import synthetic as syn
from oracle import oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = {"small": dict(in_dim=24, hidden=32, out_dim=40, classes=7, W=13, H=9, seed=41, keep=1),
         "lseg": dict(in_dim=128, hidden=128, out_dim=512, classes=20, W=20, H=19, seed=42, keep=16)}


def case_inputs(c):
    w, text = syn.make_decoder(c["in_dim"], c["hidden"], c["out_dim"], c["classes"], seed=c["seed"])
    x = syn.make_feature_map(c["W"], c["H"], c["in_dim"], seed=c["seed"] + 100)
    return w, text, x


@pytest.mark.parametrize("tag", list(CASES))
def test_oracle_decoder_and_query_equal_reference(tag):
    fx = np.load(os.path.join(HERE, "golden", "decoder.npz"))
    c = CASES[tag]
    w, text, x = case_inputs(c)
    y = orc.decode_features(x, w)
    assert y.shape == (c["H"], c["W"], c["out_dim"])
    assert np.abs(y[..., ::c["keep"]] - fx[f"{tag}_decoded"]).max() <= 2e-6      # FP32, summation order only
    labels, margin = orc.classify_features(y, text)
    ref = fx[f"{tag}_labels"]
    differ = labels != ref
    assert not differ[margin > 1e-6].any() and differ.mean() <= 0.01


def test_oracle_query_edge_cases():
    text = np.array([[1.0, 0.0], [0.0, 2.0], [0.0, 2.0]], np.float32)
    feat = np.array([[0.0, 0.0], [3.0, 1.0], [1.0, 3.0], [-1.0, -1.0]], np.float32)
    labels, margin = orc.classify_features(feat, text)
    # an all-zero row and exact ties take the first maximum, like torch.argmax on equal logits
    assert labels.tolist() == [0, 0, 1, 0] and margin[2] == 0.0
    one, m1 = orc.classify_features(feat, text[:1])
    assert one.tolist() == [0, 0, 0, 0] and (m1 == 0).all()


def test_low_precision_model_is_close_to_fp32():
    c = CASES["small"]
    w, text, x = case_inputs(c)
    a, b = orc.decode_features(x, w), orc.decode_features(x, w, precision=1)
    assert 0 < np.abs(a - b).max() < 5e-3


def test_mirror_argument_checks_need_no_device():
    from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder, classify_feature_map
    with pytest.raises(ValueError, match="feature_hwc must be 3D"):
        classify_feature_map(torch.zeros(4, 8), torch.zeros(3, 8))
    with pytest.raises(ValueError, match="text_feature must be 2D"):
        classify_feature_map(torch.zeros(2, 2, 8), torch.zeros(8))
    with pytest.raises(ValueError, match="Feature dim mismatch"):
        classify_feature_map(torch.zeros(2, 2, 8), torch.zeros(3, 9))
    with pytest.raises(RuntimeError, match="no CPU path"):
        classify_feature_map(torch.zeros(2, 2, 8), torch.zeros(3, 8))
    dec = FeatureUpsampleDecoder(24, 40, 32, device="cpu")
    w, _ = syn.make_decoder(24, 32, 40, seed=1)
    sd = {k: torch.from_numpy(v) for k, v in w.items()}
    with pytest.raises(KeyError):
        dec.load_state_dict({k: v for k, v in sd.items() if k != "net.4.bias"})
    with pytest.raises(ValueError, match="size mismatch for net.2.weight"):
        dec.load_state_dict({**sd, "net.2.weight": torch.zeros(32, 32, 1, 1)})
    with pytest.raises(KeyError, match="net.0.weight"):
        FeatureUpsampleDecoder.from_state_dict({"net.2.weight": torch.zeros(1)})
    with pytest.raises(RuntimeError, match="no CPU path"):
        FeatureUpsampleDecoder(24, 40, 32, device="cpu").decode_hwc(torch.zeros(2, 2, 24))
    with pytest.raises(ValueError, match="feature map must be"):
        FeatureUpsampleDecoder(24, 40, 32, device="cpu").decode_hwc(torch.zeros(2, 2, 25))
