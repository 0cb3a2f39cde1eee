"""Multi-GPU plumbing: one process per GPU, scene parameters replicated, frames sharded by view.

Rendering needs no per-frame exchange: tiles are independent given the parameters, views are
independent, and every frame stays on the device that rendered it.  The only collective is the
one-time broadcast of the scene's parameter tensors from rank 0 (NCCL over NVLink on GPUs, gloo on
CPU for tests).  The reference has no multi-GPU path to mirror.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

SCENE_KEYS = ("positions", "log_scales", "quats", "W1", "b1", "W2", "b2", "W3", "b3", "freq", "att", "feat_attr")


def views_for_rank(num_views: int, world_size: int, rank: int) -> list[int]:
    """Round-robin assignment of view indices to ranks."""
    return list(range(rank, num_views, world_size))


def tile_rows_for_rank(num_tile_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous band [r0, r1) of tile rows for this rank (bands differ by at most one row)."""
    base, extra = divmod(num_tile_rows, world_size)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def assign(num_views: int, num_tile_rows: int, world_size: int, rank: int):
    """Shard by view first, then by tile-row band when there are fewer views than ranks.

    Returns a list of (view, row_begin, row_end) work units for this rank.
    """
    if num_views >= world_size:
        return [(v, 0, num_tile_rows) for v in views_for_rank(num_views, world_size, rank)]
    per_view = world_size // num_views          # ranks cooperating on one view
    view, sub = rank // per_view, rank % per_view
    if view >= num_views:
        return []
    r0, r1 = tile_rows_for_rank(num_tile_rows, per_view, sub)
    return [(view, r0, r1)]


def broadcast_scene(scene: dict | None, device, src: int = 0) -> dict:
    """Broadcast a scene dict of float32 arrays from `src`; returns torch tensors on `device`.

    Shapes travel first as a small int64 tensor so that only rank `src` needs the scene.
    """
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return {k: torch.as_tensor(v).to(device) for k, v in scene.items() if k in SCENE_KEYS and v is not None}
    rank = dist.get_rank()
    meta = torch.zeros((len(SCENE_KEYS), 4), dtype=torch.int64, device=device)
    if rank == src:
        for i, k in enumerate(SCENE_KEYS):
            v = scene.get(k)
            if v is not None:
                shp = list(np.shape(v))
                meta[i, 0] = len(shp)
                for j, s in enumerate(shp):
                    meta[i, 1 + j] = s
    dist.broadcast(meta, src)
    out = {}
    meta_h = meta.cpu().tolist()
    for i, k in enumerate(SCENE_KEYS):
        nd = meta_h[i][0]
        if nd == 0:
            continue
        shape = meta_h[i][1:1 + nd]
        if rank == src:
            t = torch.as_tensor(scene[k]).to(device=device, dtype=torch.float32).contiguous()
        else:
            t = torch.empty(shape, dtype=torch.float32, device=device)
        dist.broadcast(t, src)
        out[k] = t
    return out
