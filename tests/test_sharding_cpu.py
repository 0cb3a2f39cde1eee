"""Host-side multi-GPU logic on CPU: gloo, world_size 2 (scene broadcast, work assignment)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mlp_splatting_b200 import sharding, synthetic as syn
    scene = syn.make_scene(64, seed=5, feat_dim=8) if rank == 0 else None
    got = sharding.broadcast_scene(scene, torch.device("cpu"), src=0)
    ref = syn.make_scene(64, seed=5, feat_dim=8)
    ok = all(np.array_equal(got[k].numpy(), ref[k]) for k in sharding.SCENE_KEYS)
    units = sharding.assign(num_views=4, num_tile_rows=85, world_size=world, rank=rank)
    out[rank] = (ok, units)
    dist.barrier()
    dist.destroy_process_group()


def test_broadcast_and_assignment_gloo_world2():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert out[0][0] and out[1][0]
    assert out[0][1] == [(0, 0, 85), (2, 0, 85)] and out[1][1] == [(1, 0, 85), (3, 0, 85)]


def test_assignment_covers_every_tile_row_once():
    from mlp_splatting_b200 import sharding
    for views, world in [(1, 8), (2, 8), (4, 8), (4, 2), (32, 8), (1, 1), (3, 8)]:
        cover = {}
        for r in range(world):
            for v, r0, r1 in sharding.assign(views, 85, world, r):
                for row in range(r0, r1):
                    cover[(v, row)] = cover.get((v, row), 0) + 1
        assert set(cover.values()) == {1} and len(cover) == views * 85, (views, world)


def _gather_worker(rank, world, port, out):
    """The side measurements of bench.py with several ranks: every rank brings its own record (one of them a failure),
    the only collective is the gather at the end, and rank 0 puts the records together."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    mine = {"stress": {"frames_per_sec": 0.0, "ms_per_step": 0.0, "steps": 2, "views_per_step": 32, "status_bits": 0,
                       "local": {"dev_ms": 100.0 + 50.0 * rank, "records": 1000.0 * (rank + 1), "work_total": 10.0, "work_small": 2.0}},
            "fourview": ({"failed": "RuntimeError: rank-local failure"} if rank == 1 else
                         {"frames_per_sec": 0.0, "ms_per_step": 0.0, "steps": 5, "views_per_step": 4, "status_bits": 0,
                          "local": {"dev_ms": 10.0, "records": 1.0, "work_total": 1.0, "work_small": 0.0}})}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    out[rank] = bench.combine_other_workloads(gathered) if rank == 0 else None
    dist.barrier()
    dist.destroy_process_group()


def test_side_measurements_are_gathered_once_gloo_world2():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_gather_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = out[0]
    assert res["stress"]["ms_per_step"] == 75.0 and res["stress"]["records_per_step"] == 3000.0
    assert res["stress"]["frames_per_sec"] == 32 * 2 / 0.150
    assert "rank 1: RuntimeError: rank-local failure" in res["fourview"]["failed"]
