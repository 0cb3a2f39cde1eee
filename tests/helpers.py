"""Shared test plumbing: build a seeded scene + camera and run it through the CPU oracle."""
from __future__ import annotations

import numpy as np

from mlp_splatting_b200 import synthetic as syn
from oracle import oracle as orc

WKEYS = ("W1", "b1", "W2", "b2", "W3", "b3")


def oracle_inputs(scene, cam):
    """Normalised quats/rays and packed geometry, as the renderer prepares them."""
    q = orc.normalize_rows(scene["quats"])
    rd = orc.normalize_rows(cam["rays_d"])
    geom = orc.pack_geometry(scene["positions"], scene["log_scales"], q)
    return geom, rd


def oracle_frame(scene, cam, thr, precision=0, tile=8, capacity=1536, want_records=False, feat=False,
                 want_masks=True, key_mode=0):
    """bin -> validate -> sort -> render on the CPU oracle; returns a dict of every stage's output."""
    W, H = cam["W"], cam["H"]
    geom, rd = oracle_inputs(scene, cam)
    prims, off = orc.bin_tiles(geom, cam["view"], cam["proj"], W, H, tile, thr)
    bits, mx = orc.validate_lists(off, prims, capacity, geom.shape[0])
    out = dict(geom=geom, rays_d_unit=rd, tile_prims=prims, tile_offsets=off, status=(bits, mx))
    if bits:
        return out
    sp, keys = orc.sort_tiles(cam["rays_o"], rd, geom, off, prims, W, H, tile, want_keys=True, key_mode=key_mode)
    res = orc.render(cam["rays_o"], rd, geom, off, sp, W, H, tile, thr, [scene[k] for k in WKEYS],
                     scene["freq"], scene["att"], precision=precision,
                     feat_attr=scene.get("feat_attr") if feat else None, want_masks=want_masks,
                     want_records=want_records)
    out.update(sorted_prims=sp, keys=keys, render=res)
    return out


def small_case(n=2000, W=128, H=96, mu=-3.5, seed=2026, az=0.0, hidden=32, num_freq=6, feat_dim=0):
    scene = syn.make_scene(n, seed, mu=mu, hidden=hidden, num_freq=num_freq, feat_dim=feat_dim)
    cam = syn.make_camera(W, H, azimuth_deg=az)
    return scene, cam


def popcount64(a):
    a = np.asarray(a, dtype=np.uint64)
    return np.array([bin(int(v)).count("1") for v in a], dtype=np.int64)
