"""Feature decoder and text query, same surface as scannet/feature_decoder.py and the query step of
scannet/eval_lseg_table2.py (inference only).

`FeatureUpsampleDecoder` keeps the reference's constructor, `net.{0,2,4}.{weight,bias}` state-dict keys and
NCHW `forward` (feature_decoder.py:5-19); the convolutions run in one tcgen05 kernel on the pixel-major
map the renderer writes, so `decode_hwc` is the form without permutes.  `classify_feature_map` is
`_classify_feature_map` (eval_lseg_table2.py:622-641) with the same argument checks and error texts.
`FeatureUpsampleDecoder.classify` is the two fused: the last 1x1 convolution is folded with the
normalised text embeddings when the image is packed, and the wide decoded map is never written.

There is no CPU path: every call needs a CUDA device and the built library.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L

_EYES = {}
_KEYS = ("net.0.weight", "net.0.bias", "net.2.weight", "net.2.bias", "net.4.weight", "net.4.bias")


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def classify_feature_map(feature_hwc: torch.Tensor, text_feature: torch.Tensor) -> torch.Tensor:
    """Return label map with shape [H, W], 0-based class indices (eval_lseg_table2.py:622-641)."""
    if feature_hwc.ndim != 3:
        raise ValueError(f"feature_hwc must be 3D, got {tuple(feature_hwc.shape)}")
    h, w, d = int(feature_hwc.shape[0]), int(feature_hwc.shape[1]), int(feature_hwc.shape[2])
    if text_feature.ndim != 2:
        raise ValueError(f"text_feature must be 2D, got {tuple(text_feature.shape)}")
    if int(text_feature.shape[1]) != d:
        raise ValueError(
            f"Feature dim mismatch between rendered feature ({d}) and text embedding ({int(text_feature.shape[1])}). "
            "Use matching text encoder or pass --text_feature_pt."
        )
    if not feature_hwc.is_cuda:
        raise RuntimeError("classify_feature_map runs on a CUDA device; there is no CPU path")
    lib = L.load()
    dev = feature_hwc.device
    feat = feature_hwc.reshape(-1, d).float().contiguous()
    text = text_feature.to(dev).float().contiguous()
    labels = torch.empty(h * w, device=dev, dtype=torch.int64)
    with torch.cuda.device(dev):
        L.check(lib.mlpsp_classify_features(L.ptr(feat), h * w, d, L.ptr(text), int(text.shape[0]), L.ptr(labels),
                                            _stream(dev)), "mlpsp_classify_features")
    return labels.view(h, w)


def score_labels(scores_hwc: torch.Tensor) -> torch.Tensor:
    """Per-pixel arg-max (first maximum) of a map of class scores [H, W, C], e.g. the feature map rendered from
    PackedScene.with_text_query(); labels [H, W] int64."""
    if scores_hwc.ndim != 3:
        raise ValueError(f"scores_hwc must be 3D, got {tuple(scores_hwc.shape)}")
    key = (int(scores_hwc.shape[2]), scores_hwc.device)
    eye = _EYES.get(key)
    if eye is None:
        eye = _EYES[key] = torch.eye(key[0], device=key[1], dtype=torch.float32)
    return classify_feature_map(scores_hwc, eye)


class FeatureUpsampleDecoder:
    """Feature-3DGS-style 3-layer conv decoder: 1x1 -> 3x3 -> 1x1 (feature_decoder.py:5-19), inference only."""

    def __init__(self, in_dim: int, out_dim: int, hidden_dim: int = 128, device="cuda"):
        self.in_dim, self.out_dim, self.hidden_dim = int(in_dim), int(out_dim), int(hidden_dim)
        self.device = torch.device(device)
        self._w = None
        self._packed = {}     # mode -> (image tensor, text tensor or None, text version)
        self.status = None

    # ---- state ----
    def load_state_dict(self, state_dict):
        """Accepts the reference module's state dict; `module.` / `_orig_mod.` prefixes are stripped."""
        sd = {}
        for k, v in state_dict.items():
            while k.startswith(("module.", "_orig_mod.")):
                k = k.split(".", 1)[1]
            sd[k] = v
        missing = [k for k in _KEYS if k not in sd]
        if missing:
            raise KeyError(f"Decoder checkpoint is missing {missing}")
        shapes = {"net.0.weight": (self.hidden_dim, self.in_dim, 1, 1), "net.0.bias": (self.hidden_dim,),
                  "net.2.weight": (self.hidden_dim, self.hidden_dim, 3, 3), "net.2.bias": (self.hidden_dim,),
                  "net.4.weight": (self.out_dim, self.hidden_dim, 1, 1), "net.4.bias": (self.out_dim,)}
        w = {}
        for k in _KEYS:
            t = torch.as_tensor(sd[k])
            if tuple(t.shape) != shapes[k]:
                raise ValueError(f"size mismatch for {k}: got {tuple(t.shape)}, expected {shapes[k]}")
            w[k] = t.detach().to(self.device, torch.float32).contiguous()
        self._w = w
        self._packed = {}
        if self.status is None:
            self.status = torch.zeros(L.STATUS_WORDS, device=self.device, dtype=torch.int32)
        return self

    @classmethod
    def from_state_dict(cls, state_dict, device="cuda"):
        """Sizes inferred from `net.0.weight` / `net.4.weight` as the reference's loader does
        (eval_lseg_table2.py:793-814)."""
        sd = {}
        for k, v in state_dict.items():
            while k.startswith(("module.", "_orig_mod.")):
                k = k.split(".", 1)[1]
            sd[k] = v
        w0, w4 = sd.get("net.0.weight"), sd.get("net.4.weight")
        if (not torch.is_tensor(w0)) or (not torch.is_tensor(w4)):
            raise KeyError("Decoder checkpoint is missing 'net.0.weight'/'net.4.weight'.")
        if w0.ndim != 4 or w4.ndim != 4:
            raise ValueError("Decoder checkpoint has unexpected conv weight shapes.")
        return cls(int(w0.shape[1]), int(w4.shape[0]), int(w0.shape[0]), device=device).load_state_dict(sd)

    # ---- packed images ----
    def _struct(self, text=None):
        d = L.Decoder()
        d.in_dim, d.hidden, d.out_dim = self.in_dim, self.hidden_dim, self.out_dim
        d.num_classes = 0 if text is None else int(text.shape[0])
        w = self._w
        d.W1, d.b1, d.W2, d.b2 = L.ptr(w["net.0.weight"]), L.ptr(w["net.0.bias"]), L.ptr(w["net.2.weight"]), L.ptr(w["net.2.bias"])
        d.W3, d.b3, d.text = L.ptr(w["net.4.weight"]), L.ptr(w["net.4.bias"]), L.ptr(text)
        return d

    def _image(self, mode, text=None):
        if self._w is None:
            raise RuntimeError("FeatureUpsampleDecoder has no weights: call load_state_dict first")
        hit = self._packed.get(mode)
        if hit is not None and (mode == 0 or (hit[1] is text and hit[2] == text._version)):
            return hit[0], hit[3]
        lib = L.load()
        d = self._struct(text)
        nbytes = int(lib.mlpsp_decoder_packed_bytes(C.byref(d), mode))
        if nbytes <= 0:
            raise ValueError("decoder sizes outside the kernel's limits (in_dim <= 128, hidden_dim 32/64/96/128, "
                             "at most 768 outputs or classes)")
        img = torch.empty(nbytes, device=self.device, dtype=torch.uint8)
        with torch.cuda.device(self.device):
            L.check(lib.mlpsp_pack_decoder(C.byref(d), mode, L.ptr(img), L.ptr(self.status), _stream(self.device)),
                    "mlpsp_pack_decoder")
        self._packed[mode] = (img, text, None if text is None else text._version, d)
        return img, d

    def _check_status(self, what):
        bits = int(self.status[L.ST_BITS].item())
        if bits:
            with torch.cuda.device(self.device):
                L.check(L.load().mlpsp_status_reset(L.ptr(self.status), _stream(self.device)), "mlpsp_status_reset")
            if bits & L.BIT_TIMEOUT:
                raise RuntimeError(f"{what}: a device-side wait gave up (status bit {L.BIT_TIMEOUT})")
            if bits & L.BIT_NUMERIC:
                raise FloatingPointError(f"{what}: an input, weight or activation is outside binary16 range")
            raise RuntimeError(f"{what}: status bits {bits}")

    def _map(self, feat_hwc):
        if feat_hwc.ndim != 3 or int(feat_hwc.shape[2]) != self.in_dim:
            raise ValueError(f"feature map must be [H, W, {self.in_dim}], got {tuple(feat_hwc.shape)}")
        if not feat_hwc.is_cuda:
            raise RuntimeError("the feature decoder runs on a CUDA device; there is no CPU path")
        return feat_hwc.float().contiguous()

    # ---- the three calls ----
    def decode_hwc(self, feat_hwc: torch.Tensor, check: bool = True) -> torch.Tensor:
        """decoder(feat) on a pixel-major map [H, W, in_dim] -> [H, W, out_dim]."""
        x = self._map(feat_hwc)
        h, w = int(x.shape[0]), int(x.shape[1])
        img, d = self._image(0)
        out = torch.empty((h, w, self.out_dim), device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            L.check(L.load().mlpsp_decode_features(C.byref(d), 0, L.ptr(img), L.ptr(x), w, h, L.ptr(out), None,
                                                   L.ptr(self.status), _stream(self.device)), "mlpsp_decode_features")
        if check:
            self._check_status("mlpsp_decode_features")
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[B, in_dim, H, W] -> [B, out_dim, H, W] like the reference module (feature_decoder.py:18-19)."""
        if x.ndim != 4 or int(x.shape[1]) != self.in_dim:
            raise ValueError(f"expected [B, {self.in_dim}, H, W], got {tuple(x.shape)}")
        outs = [self.decode_hwc(x[b].permute(1, 2, 0)).permute(2, 0, 1) for b in range(int(x.shape[0]))]
        return torch.stack(outs, 0) if outs else x.new_zeros((0, self.out_dim, int(x.shape[2]), int(x.shape[3])))

    __call__ = forward

    def classify(self, feat_hwc: torch.Tensor, text_feature: torch.Tensor, check: bool = True) -> torch.Tensor:
        """_classify_feature_map(decoder(feat), text) -> labels [H, W] (int64) in one kernel."""
        x = self._map(feat_hwc)
        if text_feature.ndim != 2:
            raise ValueError(f"text_feature must be 2D, got {tuple(text_feature.shape)}")
        if int(text_feature.shape[1]) != self.out_dim:
            raise ValueError(
                f"Feature dim mismatch between rendered feature ({self.out_dim}) and text embedding "
                f"({int(text_feature.shape[1])}). Use matching text encoder or pass --text_feature_pt.")
        if not (text_feature.is_cuda and text_feature.dtype == torch.float32 and text_feature.is_contiguous()):
            text_feature = text_feature.to(self.device, torch.float32).contiguous()
        h, w = int(x.shape[0]), int(x.shape[1])
        img, d = self._image(1, text_feature)
        labels = torch.empty((h, w), device=self.device, dtype=torch.int64)
        with torch.cuda.device(self.device):
            L.check(L.load().mlpsp_decode_features(C.byref(d), 1, L.ptr(img), L.ptr(x), w, h, None, L.ptr(labels),
                                                   L.ptr(self.status), _stream(self.device)), "mlpsp_decode_features")
        if check:
            self._check_status("mlpsp_decode_features")
        return labels
