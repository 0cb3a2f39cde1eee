"""Scene checkpoints on either side of the render path.

The reference saves scenes as PyTorch state dicts, bare or wrapped in a training state, with optional
``module.`` / ``_orig_mod.`` prefixes and, in old files, ``mlps.lin*`` names for the per-primitive MLP
(scannet/checkpoints.py:19-29, 69-163).  Its inference export keeps geometry in FP32 and stores the MLP
weights, biases and feature attributes in FP16 (make_inference_checkpoint, scannet/checkpoints.py:320-382);
restore_scene_state_dict (299-317) widens them again before rendering.  This module reads all of those
forms and hands the tensors to engine.PackedScene, whose packer lays the weights out for the tensor-core
evaluator, and writes the same inference export.  No renderer or CUDA dependency.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

import math

import torch

WRAPPER_KEYS = ("scene_state_dict", "state_dict")
STRIP_PREFIXES = ("module.", "_orig_mod.")
OLD_MLP_NAMES = {"mlps.lin1.weight": "W1", "mlps.lin1.bias": "b1", "mlps.lin2.weight": "W2",
                 "mlps.lin2.bias": "b2", "mlps.lin3.weight": "W3", "mlps.lin3.bias": "b3"}
MLP_KEYS = ("W1", "b1", "W2", "b2", "W3", "b3")
HALF_STORAGE = frozenset(MLP_KEYS + ("feat_attr",))
GEOMETRY = {"positions": 3, "log_scales": 3, "quats": 4}


@dataclass(frozen=True)
class SceneDims:
    num_primitives: int
    hidden_dim: int
    encoded_dim: int
    pe_frequencies: int
    feature_dim: int
    feature_slots: int


def _looks_like_scene(m: Any) -> bool:
    return isinstance(m, Mapping) and len(m) > 0 and any(
        isinstance(k, str) and k.endswith(("positions", "W1", "mlps.lin1.weight")) for k in m)


def locate_scene_state(checkpoint: Mapping[str, Any]):
    """(scene state dict, wrapper key or None) of a bare or wrapped checkpoint."""
    if not isinstance(checkpoint, Mapping):
        raise TypeError(f"checkpoint must be a mapping, got {type(checkpoint).__name__}")
    for key in WRAPPER_KEYS:
        inner = checkpoint.get(key)
        if _looks_like_scene(inner):
            return dict(inner), key
    if _looks_like_scene(checkpoint):
        return dict(checkpoint), None
    raise ValueError("could not find a scene state_dict; expected a bare scene state_dict "
                     "or a 'scene_state_dict'/'state_dict' wrapper")


def canonical_keys(state: Mapping[str, Any]) -> dict:
    """Drop wrapper prefixes and rename the old MLP parameter names; everything else is kept."""
    out: dict = {}
    for key, value in state.items():
        if not isinstance(key, str):
            raise TypeError(f"state_dict key must be str, got {type(key).__name__}")
        name = key
        stripped = True
        while stripped:
            stripped = False
            for pre in STRIP_PREFIXES:
                if name.startswith(pre):
                    name, stripped = name[len(pre):], True
        if name in out and out[name] is not value:
            raise ValueError(f"key collision after prefix removal: {key!r} -> {name!r}")
        out[name] = value
    old = [k for k in OLD_MLP_NAMES if k in out]
    if old and len(old) != len(OLD_MLP_NAMES):
        raise KeyError(f"incomplete legacy MLP state; missing {sorted(set(OLD_MLP_NAMES) - set(old))}")
    for k in old:
        new, value = OLD_MLP_NAMES[k], out.pop(k)
        if new in out and out[new] is not value:
            cur = out[new]
            same = torch.is_tensor(cur) and torch.is_tensor(value) and cur.shape == value.shape and torch.equal(cur, value)
            if not same:
                raise ValueError(f"both legacy key {k!r} and canonical key {new!r} differ")
        else:
            out[new] = value
    return out


def _need(state, key):
    t = state.get(key)
    if not torch.is_tensor(t):
        raise KeyError(f"required tensor {key!r} is missing")
    return t


def scene_dims(state: Mapping[str, Any]) -> SceneDims:
    """N, hidden width, encoded width and feature layout, with every shape checked against them."""
    s = canonical_keys(state)
    w1 = _need(s, "W1")
    if w1.ndim != 3:
        raise ValueError(f"W1 must have shape [N,H,encoded_dim], got {tuple(w1.shape)}")
    n, h, e = (int(v) for v in w1.shape)
    if min(n, h, e) <= 0:
        raise ValueError("scene dimensions must be positive")
    if e % 12:
        raise ValueError(f"encoded_dim={e} is not divisible by 12 (6D input x sin/cos positional encoding)")
    want = {"b1": (n, h), "W2": (n, h, h), "b2": (n, h), "W3": (n, 4, h), "b3": (n, 4)}
    want.update({k: (n, c) for k, c in GEOMETRY.items()})
    for k, shape in want.items():
        if tuple(_need(s, k).shape) != shape:
            raise ValueError(f"{k} has shape {tuple(s[k].shape)}, expected {shape}")
    fdim = fslots = 0
    feat = s.get("feat_attr")
    if feat is not None:
        if not torch.is_tensor(feat):
            raise TypeError("feat_attr must be a tensor")
        if feat.ndim == 2 and int(feat.shape[0]) == n:
            fdim, fslots = int(feat.shape[1]), 1
        elif feat.ndim == 3 and int(feat.shape[0]) == n:
            fslots, fdim = int(feat.shape[1]), int(feat.shape[2])
        else:
            raise ValueError(f"feat_attr must have shape [N,D] or [N,S,D] with N={n}, got {tuple(feat.shape)}")
        if fdim <= 0 or fslots <= 0:
            raise ValueError("feature dimensions must be positive")
    return SceneDims(n, h, e, e // 12, fdim, fslots)


def fold_feature_slots(feat: torch.Tensor, target_slots: int) -> torch.Tensor:
    """Five slots hold a base and four deltas, four slots the directional embeddings themselves
    (scannet/checkpoints.py:219-245): 5 -> 4 adds the base to every delta, 4 -> 5 prepends a zero base."""
    if not torch.is_tensor(feat) or feat.ndim != 3:
        raise ValueError("feature must be a tensor with shape [N,S,D]")
    if target_slots not in (4, 5):
        raise ValueError("target_slots must be 4 or 5")
    have = int(feat.shape[1])
    if have == target_slots:
        return feat.clone()
    if (have, target_slots) == (5, 4):
        return feat[:, :1, :] + feat[:, 1:, :]
    if (have, target_slots) == (4, 5):
        return torch.cat((torch.zeros_like(feat[:, :1, :]), feat), dim=1)
    raise ValueError(f"cannot convert {have}-slot features to {target_slots} slots")


def widen_to_float32(state: Mapping[str, Any]) -> dict:
    """FP16 is a storage format for MLP weights and features only; everything floating becomes FP32."""
    s = canonical_keys(state)
    for name, v in s.items():
        if not torch.is_tensor(v) or not v.is_floating_point():
            continue
        if v.dtype == torch.float16 and name not in HALF_STORAGE:
            raise TypeError(f"{name}: FP16 storage is only supported for MLP weights and features")
        if v.dtype not in (torch.float16, torch.float32, torch.float64):
            raise TypeError(f"{name}: unsupported scene storage dtype {v.dtype}")
        s[name] = v.float()
    return s


def export_inference_state(checkpoint: Mapping[str, Any], storage_precision: str = "mixed",
                           target_feature_slots: int = 4) -> dict:
    """The reference's inference export of a checkpoint: same keys, dtypes and metadata as
    make_inference_checkpoint (scannet/checkpoints.py:320-382)."""
    if storage_precision not in ("mixed", "fp32"):
        raise ValueError("storage_precision must be mixed or fp32")
    if target_feature_slots not in (4, 5):
        raise ValueError("target_feature_slots must be 4 or 5")
    raw, wrapper = locate_scene_state(checkpoint)
    canon = canonical_keys(raw)
    for name, v in canon.items():
        if torch.is_tensor(v) and v.is_floating_point():
            ok = (torch.float16, torch.float32) if name in HALF_STORAGE else (torch.float32,)
            if v.dtype not in ok:
                raise TypeError(f"{name}: inference export requires FP32 geometry and auxiliary state")
    state = widen_to_float32({k: (v.detach().cpu().contiguous().clone() if torch.is_tensor(v) else v)
                              for k, v in canon.items()})
    dims = scene_dims(state)
    if dims.feature_slots not in (0, 4, 5):
        raise ValueError("inference export requires directional features with 4 or 5 slots, or RGB-only state")
    if dims.feature_slots in (4, 5):
        state["feat_attr"] = fold_feature_slots(state["feat_attr"], target_feature_slots)
    out_state = {}
    for name, v in state.items():
        if not torch.is_tensor(v):
            raise TypeError(f"{name}: scene state entries must be tensors")
        v = v.detach().contiguous()
        if v.is_floating_point():
            if not bool(torch.isfinite(v).all()):
                raise ValueError(f"{name}: cannot export non-finite values")
            if storage_precision == "mixed" and name in HALF_STORAGE:
                v = v.half()
                if not bool(torch.isfinite(v).all()):
                    raise ValueError(f"{name}: values overflow FP16 storage")
        out_state[name] = v
    after = scene_dims(out_state)
    out = dict(checkpoint) if wrapper else {}
    out[wrapper or "scene_state_dict"] = out_state
    out.pop("optimizer_state_dict", None)
    meta = dict(out.get("metadata", {}))
    meta.update(inference_only=True,
                storage_precision=("float16_mlp_and_features_float32_geometry" if storage_precision == "mixed" else "float32"),
                feature_slots=after.feature_slots, feature_dim=after.feature_dim)
    if after.feature_slots in (4, 5):
        meta["feature_slot_layout"] = "direct_tetrahedral" if after.feature_slots == 4 else "legacy_base_plus_four_deltas"
    if "feature_dim_low" in meta:
        meta["feature_dim_low"] = after.feature_dim
    out["metadata"] = meta
    for name, value in (("feature_slots", after.feature_slots), ("feature_dim_low", after.feature_dim)):
        if name in out:
            out[name] = value
    return out


def scene_arrays(checkpoint: Mapping[str, Any], pe_sigma: float = 0.01, integrated: bool = True) -> dict:
    """Float32 tensors of a checkpoint under the names engine.PackedScene takes, plus freq / att.

    The encoder's bands come from the checkpoint when it carries them (``encoder.freq_bands``), else they
    are rebuilt as the reference builds them (scannet/cumodel.py:138, 163): 2^k * pi with attenuation
    exp(-f^2 sigma^2 / 2) for the integrated encoder, 2^k unattenuated for the Fourier one."""
    raw, _ = locate_scene_state(checkpoint)
    s = widen_to_float32(raw)
    dims = scene_dims(s)
    out = {k: s[k].contiguous() for k in ("positions", "log_scales", "quats") + MLP_KEYS}
    if dims.feature_slots:
        out["feat_attr"] = s["feat_attr"].contiguous()
    bands = s.get("encoder.freq_bands")
    if torch.is_tensor(bands) and bands.numel() == dims.pe_frequencies:
        freq = bands.float().reshape(-1)
    else:
        freq = 2.0 ** torch.arange(dims.pe_frequencies, dtype=torch.float32)
        if integrated:
            freq = freq * math.pi
    att = torch.exp(-0.5 * freq * freq * float(pe_sigma) ** 2) if integrated else torch.ones_like(freq)
    out["freq"], out["att"] = freq, att
    return out


def load_packed_scene(path_or_checkpoint, device, pe_sigma: float = 0.01, integrated: bool = True, pack_f16: bool = True):
    """Read a checkpoint (path or mapping) straight into an engine.PackedScene on `device`."""
    from .engine import PackedScene
    ckpt = path_or_checkpoint
    if not isinstance(ckpt, Mapping):
        ckpt = torch.load(ckpt, map_location="cpu", weights_only=True)
    a = scene_arrays(ckpt, pe_sigma=pe_sigma, integrated=integrated)
    return PackedScene(a["positions"], a["log_scales"], a["quats"], *[a[k] for k in MLP_KEYS], a["freq"], a["att"],
                       feat_attr=a.get("feat_attr"), device=device, pack_f16=pack_f16)


def scene_module_from_checkpoint(path_or_checkpoint, device=None, **module_kwargs):
    """Build a cumodel.NeuralPrimitiveSceneTileCUDA of the checkpoint's dimensions and load its tensors, the
    way the reference's evaluation scripts do (scannet/eval_rgb_psnr.py:156-235: infer the spec, construct
    the scene, load the restored state dict)."""
    from .cumodel import NeuralPrimitiveSceneTileCUDA
    ckpt = path_or_checkpoint
    if not isinstance(ckpt, Mapping):
        ckpt = torch.load(ckpt, map_location="cpu", weights_only=True)
    raw, _ = locate_scene_state(ckpt)
    state = widen_to_float32(raw)
    d = scene_dims(state)
    kw = dict(num_primitives=d.num_primitives, hidden_dim=d.hidden_dim, pe_frequencies=d.pe_frequencies,
              feature_dim_low=d.feature_dim, feature_slots=d.feature_slots if d.feature_slots else 4)
    kw.update(module_kwargs)
    scene = NeuralPrimitiveSceneTileCUDA(**kw)
    own = scene.state_dict()
    missing = [k for k, _ in scene.named_parameters() if k not in state]
    if missing:
        raise KeyError(f"checkpoint lacks {missing}")
    scene.load_state_dict({k: v for k, v in state.items() if k in own}, strict=False)
    return scene.to(device) if device is not None else scene
