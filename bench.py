"""Benchmark of the render hot path: frames/s (and record-MLP evaluations/s) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one frame of the named workload through the whole path (binning, per-tile sort, record
waves with the per-primitive MLP, compositing).  `value` is whole-job frames/s with the scene and
the rays resident in HBM; `e2e` is the same frame through the public host API with the rays
arriving from pinned host memory and the image returning to it inside the timed region.  At N > 1
every rank renders its own view of the replicated scene (weak scaling); the scene is generated on
rank 0 and broadcast once with NCCL.  `--impl reference` times the CPU restatement of the
reference's algorithm (oracle/) on the host cores over a bounded band of tile rows.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WK = ("W1", "b1", "W2", "b2", "W3", "b3")
FLOP_PER_RECORD = 6912          # 2*(72*32 + 32*32 + 32*4): algorithmic MLP work of one record (hidden 32)


def flop_per_record(hidden):
    return 2 * (72 * hidden + hidden * hidden + hidden * 4)     # 17,920 at hidden 64
THRESHOLD = 5e-3                # score threshold of the reference's benchmark tool


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Number of samples taken so far (marks the start of a window)."""
        return len(self.lines)

    def stop(self, first=0):
        """Summary of the samples from index `first` on."""
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines[first:]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        hot = [s for s in sm if s > 0.5 * (max(sm) if sm else 1)]
        return dict(sm_mhz=statistics.median(hot) if hot else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def cpu_baseline(scene, cam, budget_s, steps=1, warmup=0):
    """Oracle (CPU restatement of the reference algorithm) on a band of tile rows; frames/s scaled to a frame."""
    from oracle import oracle as orc
    W, H = cam["W"], cam["H"]
    ntx, nty = (W + 7) // 8, (H + 7) // 8
    q = orc.normalize_rows(scene["quats"])
    rd = orc.normalize_rows(cam["rays_d"])
    geom = orc.pack_geometry(scene["positions"], scene["log_scales"], q)
    weights = [scene[k] for k in WK]

    def frame(rows):
        r0 = (nty - rows) // 2
        t0 = time.perf_counter()
        prims, off = orc.bin_tiles(geom, cam["view"], cam["proj"], W, H, 8, THRESHOLD)
        sp = orc.sort_tiles(cam["rays_o"], rd, geom, off, prims, W, H, 8)
        res = orc.render(cam["rays_o"], rd, geom, off, sp, W, H, 8, THRESHOLD, weights, scene["freq"], scene["att"],
                         precision=1, want_masks=False, tile_range=(r0 * ntx, (r0 + rows) * ntx))
        return time.perf_counter() - t0, res.evals

    probe_rows = max(1, nty // 24)
    dt, _ = frame(probe_rows)
    rows = int(max(1, min(nty, probe_rows * budget_s / max(dt, 1e-6))))
    times, evals = [], 0
    for i in range(warmup + steps):
        dt, ev = frame(rows)
        if i >= warmup:
            times.append(dt); evals += ev
    mean = sum(times) / len(times)
    frac = rows / nty
    return dict(value=frac / mean, unit="frames/s", cores=orc.num_threads(), kind="port",
                sample=f"{rows} of {nty} tile rows ({frac:.3f} of a frame; binning and sort of the whole frame included), "
                       f"{len(times)} timed pass(es) of {mean:.2f} s, fp16-operand MLP model, OpenMP over tiles",
                evals_per_s=evals / sum(times), ms_per_step=mean * 1e3)


def reference_cuda_kernels(scene, cam, steps):
    """Device time of the reference's own CUDA kernels (compiled unmodified for sm_100a by oracle/build_ref.py)
    on this workload, given tile lists from the oracle's binning.  Extra evidence only: the reference arm's
    value stays the CPU number.  Returns None when the module or a GPU is missing."""
    try:
        import torch
        from oracle import build_ref
        from oracle import oracle as orc
        if not torch.cuda.is_available():
            return None
        mod = build_ref.load_module()
        if mod is None:
            return None
        dev = torch.device("cuda", 0)
        W, H = cam["W"], cam["H"]
        q = orc.normalize_rows(scene["quats"])
        rd = orc.normalize_rows(cam["rays_d"])
        geom = orc.pack_geometry(scene["positions"], scene["log_scales"], q)
        prims, off = orc.bin_tiles(geom, cam["view"], cam["proj"], W, H, 8, THRESHOLD)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        x = [t(cam["rays_o"]), t(rd), t(scene["positions"]), t(scene["log_scales"]), t(q), t(prims), t(off),
             t(scene["freq"]), t(scene["att"])] + [t(scene[k]) for k in WK]
        out = {"note": "reference kernels, unmodified, sm_100a build; culling (dense PyTorch in the reference) not "
                       "included; CUDA events, L2 not flushed"}
        for name, call in (("render_tiles_forward_tilecenter", lambda: mod.render_tiles_forward_tilecenter(*x, W, H, 8, 8, THRESHOLD)),
                           ("render_tiles_rgb_wmma_f16", lambda: mod.render_tiles_rgb_wmma(x, W, H, THRESHOLD, False))):
            for _ in range(2):
                call()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(max(1, steps)):
                call()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / max(1, steps)
            out[name] = {"ms_per_frame": ms, "frames_per_s": 1e3 / ms}
        return out
    except Exception as exc:   # evidence only: never fail the arm over it
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mlp_splatting_b200 import synthetic as syn
    scene, cams, cfg = syn.make_workload(args.workload)
    per_step = max(2.0, 150.0 / (args.steps + args.warmup + 1))
    cb = cpu_baseline(scene, cams[0], per_step, steps=args.steps, warmup=args.warmup)
    ref_gpu = reference_cuda_kernels(scene, cams[0], min(args.steps, 5))
    line = {
        "impl": "reference", "metric": "frames_per_sec", "value": cb["value"], "unit": "frames/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(args.workload, cfg, 1, args.encoder),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "record_mlp_evals_per_sec": cb["evals_per_s"],
    }
    if ref_gpu is not None:
        line["reference_cuda_kernels"] = ref_gpu
    print(json.dumps(line), flush=True)


def workload_config(name, cfg, n_gpus, encoder="integrated"):
    views = int(cfg["views"])
    return {"workload": name, "encoder": encoder, "primitives": cfg["n"], "width": cfg["W"], "height": cfg["H"], "tile": 8,
            "tile_capacity": 1536, "threshold": THRESHOLD, "log_scale_mean": cfg["mu"],
            "mlp": f"72-{cfg.get('hidden', 32)}-{cfg.get('hidden', 32)}-4 fp16 weights, fp32 accumulate", "views_per_step": n_gpus if views == 1 else views,
            "feature_channels": cfg.get("feat_dim", 0),
            "after_feature_map": (f"decoder {cfg['feat_dim']}-{cfg['decoder']['hidden']}-{cfg['decoder']['out_dim']} (1x1, 3x3, 1x1) + "
                                  f"{cfg['decoder']['classes']}-class text query, labels per pixel; not part of the e2e arm"
                                  if cfg.get("decoder") else
                                  (f"{cfg['text_query']['classes']}-class text query by projecting the scene's features onto the "
                                   "normalised embeddings once; class scores composited, labels per pixel; not part of the e2e arm"
                                   if cfg.get("text_query") else None)),
            "parallelism": (f"one view per GPU x{n_gpus} (azimuth 90 deg x (rank mod 4))" if views == 1 else f"{views} views shared by {n_gpus} GPU(s) by view, then by tile-row band")
                           + ", scene replicated",
            "l2": "256 MB flush between timed steps"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="single_100k_1200x680")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="fp16", choices=["fp16", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--encoder", default="integrated", choices=["integrated", "fourier"],
                    help="integrated: the reference default (bands attenuated by exp(-f^2 sigma^2 / 2), sigma 0.01); "
                         "fourier: unattenuated power-of-two bands")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from mlp_splatting_b200 import _lib as L
    from mlp_splatting_b200 import sharding, synthetic as syn
    from mlp_splatting_b200.engine import FrameRenderer, PackedScene

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the render path has no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    cfg = dict(syn.WORKLOADS[args.workload])
    scene_np = None
    if rank == 0:
        scene_np = syn.make_scene(cfg["n"], cfg["seed"], mu=cfg["mu"], hidden=cfg.get("hidden", 32),
                                  feat_dim=cfg.get("feat_dim", 0), pe_sigma=0.01 if args.encoder == "integrated" else 0.0)
    t_b0 = time.perf_counter()
    scene_t = sharding.broadcast_scene(scene_np, dev, src=0)
    torch.cuda.synchronize()
    bcast_s = time.perf_counter() - t_b0
    prec = L.PRECISION_F16 if args.precision == "fp16" else L.PRECISION_F32
    ps = PackedScene(*[scene_t[k] for k in ("positions", "log_scales", "quats") + WK], scene_t["freq"], scene_t["att"],
                     feat_attr=scene_t.get("feat_attr"), device=dev, pack_f16=(prec == L.PRECISION_F16))
    # Work units of this rank.  Single-view workloads: one view per rank on the circle of radius 3 (weak
    # scaling, per-GPU work fixed).  Multi-view workloads: the workload's views are shared between the
    # ranks, by view and then by band of tile rows (strong scaling, total work fixed).
    nviews = int(cfg["views"])
    nty = (cfg["H"] + 7) // 8
    want_feat = cfg.get("feat_dim", 0) > 0
    if nviews == 1:
        # face-on views only (0/90/180/270 degrees): seen along a diagonal the same cube puts more than
        # 1,536 candidates into some tiles, which the path rejects exactly as the reference does
        units = [(syn.make_camera(cfg["W"], cfg["H"], azimuth_deg=90.0 * (rank % 4)), None)]
        frames_per_step, scaling = world, "weak"
    else:
        units = [(syn.make_camera(cfg["W"], cfg["H"], azimuth_deg=360.0 * v / nviews), (r0, r1) if (r0, r1) != (0, nty) else None)
                 for v, r0, r1 in sharding.assign(nviews, nty, world, rank)]
        frames_per_step, scaling = nviews, "strong"
    cam = units[0][0] if units else syn.make_camera(cfg["W"], cfg["H"])
    r = FrameRenderer(cfg["W"], cfg["H"], device=dev)
    dev_rays = []
    for c, _rows in units:
        rd_dev = torch.from_numpy(c["rays_d"]).to(dev)
        rd_u = torch.empty_like(rd_dev)
        L.check(lib.mlpsp_normalize_rows(L.ptr(rd_dev), L.ptr(rd_u), r.P, 3, None), "normalize")
        dev_rays.append((torch.from_numpy(c["rays_o"]).to(dev), rd_u))
    ro_h = torch.from_numpy(cam["rays_o"]).pin_memory()
    rd_h = torch.from_numpy(cam["rays_d"]).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    # the step after the feature map, for workloads that name a decoder: decoder + text query in one kernel
    dec = text = labels = None
    if cfg.get("decoder"):
        from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder
        dc = cfg["decoder"]
        dw, dtext = syn.make_decoder(cfg["feat_dim"], dc["hidden"], dc["out_dim"], dc["classes"], seed=dc["seed"])
        dec = FeatureUpsampleDecoder(cfg["feat_dim"], dc["out_dim"], dc["hidden"], device=dev)
        dec.load_state_dict({k: torch.from_numpy(v) for k, v in dw.items()})
        text = torch.from_numpy(dtext).to(dev)

    score_dim = 0
    if cfg.get("text_query"):
        from mlp_splatting_b200.feature_decoder import score_labels
        tq = cfg["text_query"]
        qtext = torch.from_numpy(np.random.default_rng(tq["seed"]).normal(size=(tq["classes"], cfg["feat_dim"])).astype(np.float32))
        ps = ps.with_text_query(qtext)
        score_dim = tq["classes"]

    def frame(check=False):
        nonlocal labels
        out = None
        for (c, rows), (ro_u, rd_u) in zip(units, dev_rays):
            out = r.render(ps, ro_u, rd_u, THRESHOLD, view=c["view"], proj=c["proj"], precision=prec,
                           rays_normalized=True, check=check, tile_rows=rows, want_feat=want_feat)
            if dec is not None:
                labels = dec.classify(r.feat.view(cfg["H"], cfg["W"], cfg["feat_dim"]), text, check=check)
            if score_dim:
                labels = score_labels(r.feat.view(cfg["H"], cfg["W"], score_dim))
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # sizing pass (grows scratch if needed), then warm-up
    frame(check=True)
    stats = r.last_stats
    if nviews > 1:   # per-step totals over this rank's units
        tot_rec = tot_used = 0
        for (c, rows), (ro_u, rd_u) in zip(units, dev_rays):
            r.render(ps, ro_u, rd_u, THRESHOLD, view=c["view"], proj=c["proj"], precision=prec, rays_normalized=True,
                     tile_rows=rows, want_feat=want_feat)
            tot_rec += r.last_stats.records; tot_used += r.last_stats.used
        stats.records, stats.used = tot_rec, tot_used
    for _ in range(args.warmup):
        flush.fill_(1); frame()
    barrier()

    # ---- timed region: K frames, device time per frame by CUDA events, L2 flushed between frames ----
    clock_mark = sampler.mark()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = lib.mlpsp_kernel_launches(None, 0)
    barrier()
    wall0 = time.perf_counter()
    for a, b in evs:
        flush.fill_(1)
        a.record(); frame(); b.record()
    barrier()
    wall = time.perf_counter() - wall0
    launches = lib.mlpsp_kernel_launches(None, 0) - launches0
    dev_ms = sum(a.elapsed_time(b) for a, b in evs)
    # nvidia-smi answers every 20-100 ms and the timed region may be shorter than that: the same frames keep
    # running (untimed) until the window that opened with the timed region holds a handful of samples
    clock_extra = 0
    if rank == 0 and sampler.proc is not None:
        t_c = time.perf_counter()
        while sampler.mark() - clock_mark < 5 and time.perf_counter() - t_c < 1.5:
            frame(); torch.cuda.synchronize(); clock_extra += 1
    clocks = sampler.stop(clock_mark) if rank == 0 else None
    if clocks is not None:
        clocks["window"] = f"timed region + {clock_extra} further untimed frames of the same workload"
    barrier()
    bits = int(r.status.cpu()[0])
    if bits & ~L.BIT_NUMERIC:
        raise SystemExit(f"render status bits {bits} during the timed region")
    t = torch.tensor([dev_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms_max = float(t.item())
    ms_per_step = dev_ms_max / args.steps
    fps = frames_per_step * args.steps / (dev_ms_max / 1e3)
    rec_t = torch.tensor([float(stats.records), float(stats.used)], dtype=torch.float64, device=dev)
    if world > 1 and nviews > 1:
        dist.all_reduce(rec_t)   # records of the whole step (all views), summed over ranks

    # ---- per-kernel-class device time (separate pass: event pairs around every launch group) ----
    lib.mlpsp_timing_enable(1)
    per_class0 = (C.c_int64 * 8)()
    lib.mlpsp_kernel_launches(per_class0, 8)
    tsteps = min(args.steps, 10)
    for _ in range(tsteps):
        flush.fill_(1); frame()
    torch.cuda.synchronize()
    ms_cls = (C.c_float * 8)()
    L.check(lib.mlpsp_timing_collect(ms_cls, 8), "timing_collect")
    lib.mlpsp_timing_enable(0)
    per_class1 = (C.c_int64 * 8)()
    lib.mlpsp_kernel_launches(per_class1, 8)
    classes = {}
    for i, name in enumerate(L.KERNEL_CLASSES):
        n_l = (per_class1[i] - per_class0[i]) / tsteps
        classes[name] = {"ms_per_step": ms_cls[i] / tsteps, "launches_per_step": n_l}
    pk = peaks()
    mlp_ms = classes["mlp"]["ms_per_step"]
    mlp_launch_ms = mlp_ms / max(classes["mlp"]["launches_per_step"], 1)
    hidden = int(cfg.get("hidden", 32))
    flops_step = stats.records * flop_per_record(hidden)
    achieved_tf = flops_step / (mlp_ms / 1e3) / 1e12 if mlp_ms > 0 else 0.0
    roofline = {"kernel": "k_mlp_tc (per-primitive MLP, tcgen05)", "bound": "tensor", "achieved": achieved_tf,
                "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved_tf / pk["bf16_tflops"],
                "peak_source": pk["source"] + " burst", "traffic": None,
                "flop_per_launch": flops_step / max(classes["mlp"]["launches_per_step"], 1),
                "avg_launch_ms": mlp_launch_ms, "share_of_step": mlp_ms / max(sum(c["ms_per_step"] for c in classes.values()), 1e-9)}
    # Algorithmic bytes of the evaluator: 32 B in + 16 B out per record, one 8,464-byte weight image per work item.
    n_launch = max(classes["mlp"]["launches_per_step"], 1)
    alg_bytes = stats.records * 48 + stats.work_total * (8464 if hidden == 32 else 21008)
    roofline["hbm_view"] = {"algorithmic_bytes_per_launch": alg_bytes / n_launch,
                            "achieved_gbs": alg_bytes / (mlp_ms / 1e3) / 1e9 if mlp_ms > 0 else 0.0,
                            "peak_gbs": pk["hbm_gbs"],
                            "frac": (alg_bytes / (mlp_ms / 1e3) / 1e9 / pk["hbm_gbs"]) if mlp_ms > 0 else 0.0}
    if args.workload == "single_100k_1200x680" and prec == L.PRECISION_F16 and args.encoder == "integrated" and nviews == 1:
        # one ncu capture of the three busy evaluator launches of a frame of this workload: DRAM read + write bytes
        # 386.7 + 272.7 + 86.5 MB; the other launches of the six-wave schedule move nothing
        roofline["traffic"] = (386.7e6 + 272.7e6 + 86.5e6) / n_launch
        roofline["traffic_unit"] = "bytes per launch: ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over a frame's evaluator launches"
        roofline["ncu_pipes_pct"] = {"tensor": 10.2, "special_function": 48.0, "issue": 57.0, "dram": 16.6,
                                     "source": "profiles/k_mlp_tc_single_100k_1200x680.md (largest wave)"}

    # ---- end to end: pinned host rays in, image out, status checked, through the public host API.
    # Three frames are kept in flight (FramePipeline): every step still copies its own rays to the device
    # and its own image back inside the timed region; the copies of one frame overlap the kernels of others.
    from mlp_splatting_b200.engine import FramePipeline
    depth = 3
    pipe = FramePipeline(ps, cfg["W"], cfg["H"], depth=depth, max_records=r.max_records)
    outs = [(torch.empty((r.P, 3), dtype=torch.float32).pin_memory(), torch.empty((r.P, 1), dtype=torch.float32).pin_memory())
            for _ in range(depth)]

    host_rays = [(torch.from_numpy(c["rays_o"]).pin_memory(), torch.from_numpy(c["rays_d"]).pin_memory()) for c, _ in units]

    def e2e_run(k):
        j = 0
        for _i in range(k):
            for (c, rows), (roh, rdh) in zip(units, host_rays):
                o = outs[j % depth]; j += 1
                pipe.submit(roh, rdh, THRESHOLD, c["view"], c["proj"], out_rgb_host=o[0], out_alpha_host=o[1],
                            precision=prec, tile_rows=rows)
        pipe.drain()

    e2e_run(2 * depth)
    barrier()
    e0 = time.perf_counter()
    e2e_run(args.steps)
    barrier()
    e_t = torch.tensor([time.perf_counter() - e0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e_t, op=dist.ReduceOp.MAX)
    e2e_fps = frames_per_step * args.steps / float(e_t.item())
    last = (args.steps * max(len(units), 1) - 1) % depth
    e2e_err = float((outs[last][0].to(dev) - r.rgb).abs().max()) if units else 0.0   # must reproduce the resident-input frame

    if rank == 0:
        line = {
            "metric": "frames_per_sec", "value": fps, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f16" if prec == L.PRECISION_F16 else "f32", "data": "synthetic",
            "config": workload_config(args.workload, cfg, world, args.encoder),
            "record_mlp_evals_per_sec": float(rec_t[0]) * (fps / frames_per_step if nviews > 1 else fps),
            "records_per_frame": {"evaluated": stats.records, "composited": stats.used, "candidate_pairs": stats.pairs, "pairs_after_tile_pretest": stats.pairs_kept, "evaluator_blocks": stats.work_total,
                                  "waves": stats.waves, "max_tile_len": stats.max_tile_len},
            "e2e": {"value": e2e_fps, "unit": "frames/s", "h2d_bytes_per_step": 2 * r.P * 12 * max(len(units), 1),
                    "d2h_bytes_per_step": (r.P * 16 + 64) * max(len(units), 1),
                    "frames_in_flight": depth, "max_abs_diff_vs_resident_frame": e2e_err},
            "gpu_launches": int(launches),
            "kernel_classes": classes,
            "roofline": roofline,
            "clocks": clocks,
            "scene_broadcast_s": bcast_s if world > 1 else 0.0,
            "wall_ms_per_step": wall * 1e3 / args.steps,
        }
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline(scene_np, cam, budget_s=15.0)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
