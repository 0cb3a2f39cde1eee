"""Ray-cone tile culling for cameras a projection matrix cannot describe, same call as
scannet/camera.py:102-146 `ray_cone_candidates` (the COLMAP ray models and the undistortion of that
module belong to the data loaders and are not part of the render path)."""
from __future__ import annotations

import torch

from . import _lib as L
from .engine import FrameRenderer, PackedScene, RenderError


@torch.no_grad()
def ray_cone_candidates(ray_o, ray_d, positions, log_scales, width, height, tile_size, score_threshold,
                        tile_chunk=128, scene: PackedScene | None = None, renderer: FrameRenderer | None = None):
    """Conservative bound for the threshold ellipsoid using its enclosing sphere: every ray of a tile
    lies inside the tile's cone, so a primitive whose sphere misses the cone cannot be hit.
    Returns (ids int32 [M], offsets int32 [T+1]); ids ascend inside a tile."""
    if not 0 < score_threshold < 1:
        raise ValueError("score_threshold must be in (0,1)")
    if tuple(ray_o.shape) != (height * width, 3) or ray_d.shape != ray_o.shape:
        raise ValueError("ray shape mismatch")
    device = positions.device
    if ray_o.device != device or ray_d.device != device:
        raise ValueError("device mismatch")
    if device.type != "cuda":
        raise RuntimeError("ray_cone_candidates runs on a CUDA device; there is no CPU path")
    if int(tile_size) != 8:
        raise ValueError("this build renders 8x8 tiles only")
    if scene is None:
        n = positions.shape[0]
        z = torch.zeros
        q = torch.tensor([1.0, 0.0, 0.0, 0.0], device=device).repeat(n, 1)
        scene = PackedScene(positions, log_scales, q, z(n, 1, 12, device=device), z(n, 1, device=device),
                            z(n, 1, 1, device=device), z(n, 1, device=device), z(n, 4, 1, device=device),
                            z(n, 4, device=device), torch.ones(1, device=device), torch.ones(1, device=device),
                            device=device, pack_f16=False)
    r = renderer if renderer is not None else FrameRenderer(int(width), int(height), device=device)
    prims, offs, bits = r.bin_raycone(scene, ray_o.contiguous().float(), ray_d.contiguous().float(), float(score_threshold))
    if bits & L.BIT_TILE_ORIGINS:
        raise ValueError("Each tile must use a single camera origin")
    if bits & L.BIT_CONE_TOO_WIDE:
        raise ValueError("Tile ray cone spans >=90 degrees")
    return prims.clone(), offs.clone()
