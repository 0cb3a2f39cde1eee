"""Benchmark of the render hot path: frames/s (and record-MLP evaluations/s) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one frame of the named workload through the whole path (binning, per-tile sort, record
waves with the per-primitive MLP, compositing).  `value` is whole-job frames/s with the scene and
the rays resident in HBM (the first block of K timed steps; `repeat` holds median and spread over
further blocks of K steps); `e2e` is the same frame through the public host API with the rays
arriving from pinned host memory and the image returning to it inside the timed region.  At N > 1
every rank renders its own view of the replicated scene (weak scaling); the scene is generated on
rank 0 and broadcast once with NCCL.  The default one-GPU run adds, under `other_workloads`, short
measurements of the other named configurations (feature map, four views in one batch, the 2 M-primitive
stress scene in view batches, per-primitive weight gradients); with several ranks they are opt-in
(`--other-workloads-multi`, every rank measures its share without collectives, the shares are put together at the end).  `--impl reference` times the CPU restatement
of the reference's algorithm (oracle/) on all host cores over a bounded band of tile rows.
`--workload decoder_<W>x<H>` (decoder_1200x680) times the step after the feature map alone: fused decoder +
text query, decoder, full-width query (`--only` picks one).
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
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
THRESHOLD = 5e-3                # score threshold of the reference's benchmark tool
HEADLINE = "single_100k_1200x680"
OTHER_WORKLOADS = ("feature_250k_1200x680", "fourview_500k_1200x680", "stress_2m_1920x1080")


def flop_per_record(hidden):
    """Algorithmic MLP work of one record: 2*(72*H + H*H + H*4); 6,912 at H = 32, 17,920 at H = 64."""
    return 2 * (72 * hidden + hidden * hidden + hidden * 4)


def weight_image_bytes(hidden):
    """Bytes of one primitive's packed weight image (biases included), as the evaluator streams it per work item."""
    return 9472 if hidden == 32 else 22784


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def source_digest(names):
    h = {}
    for n in names:
        with open(os.path.join(ROOT, "mlp-splatting_b200", "csrc", n), "rb") as f:
            h[n] = hashlib.sha256(f.read()).hexdigest()[:16]
    return h


def ncu_figures(workload):
    """DRAM traffic and pipe utilisation of the evaluator from the ncu capture summarised under profiles/, or None
    when there is none for this workload or the kernel's sources have changed since it was taken."""
    path = os.path.join(ROOT, "profiles", f"k_mlp_tc_{workload}.json")
    if not os.path.exists(path):
        return None
    rec = json.load(open(path))
    if rec.get("sources_sha256") != source_digest(sorted(rec.get("sources_sha256", {}))):
        return None
    return rec


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

    def summary(self, first=0, last=None):
        """Summary of the samples [first, last)."""
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        sm, mx, reasons = [], [], set()
        for ln in self.lines[first:last]:
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

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


def cpu_baseline(scene, cam, budget_s, steps=1, warmup=0):
    """Oracle (CPU restatement of the reference algorithm) on a band of tile rows, on every host core this process
    may use; frames/s scaled to a frame."""
    from oracle import oracle as orc
    orc.set_num_threads(orc.host_cores())      # a launcher may have exported OMP_NUM_THREADS=1
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
    # The job of this arm at N GPUs is the job of the other arm at N GPUs (N views per step when every rank renders
    # one): the host renders the views one after the other, so its frames/s do not depend on N and one view is sampled.
    line = {
        "impl": "reference", "metric": "frames_per_sec", "value": cb["value"], "unit": "frames/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
        "scaling": "weak" if int(cfg["views"]) == 1 else "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(args.workload, cfg, args.gpus, args.encoder),
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


def packed_scene_on_device(cfg, dev, lib, chunk=131072):
    """A scene of the workload's distributions drawn on the device (synthetic.make_scene_device) and packed slice by
    slice: geometry and the fp16 weight image are kept, the FP32 weight masters of a slice are dropped once packed
    (2 M primitives with 64-wide layers would be 72 GB of masters)."""
    import torch
    from mlp_splatting_b200 import _lib as L
    from mlp_splatting_b200 import synthetic as syn
    from mlp_splatting_b200.engine import PackedScene
    n, H = int(cfg["n"]), int(cfg.get("hidden", 32))
    geo = syn.make_scene_device(n, cfg["seed"], dev, mu=cfg["mu"], hidden=H, parts=("geometry",))
    wbytes = int(lib.mlpsp_packed_weight_bytes(H, 6))
    image = torch.empty(n * wbytes, device=dev, dtype=torch.uint8)
    status = torch.zeros(L.STATUS_WORDS, device=dev, dtype=torch.int32)
    st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for a in range(0, n, chunk):
        m = min(chunk, n - a)
        part = syn.make_scene_device(m, cfg["seed"] + 1 + a, dev, hidden=H, parts=("weights",))
        s = L.Scene()
        s.n, s.hidden, s.num_freq = m, H, 6
        s.W1, s.b1, s.W2, s.b2, s.W3, s.b3 = (L.ptr(part[k]) for k in WK)
        L.check(lib.mlpsp_pack_weights_f16(C.byref(s), image.data_ptr() + a * wbytes, L.ptr(status), st), "mlpsp_pack_weights_f16")
        torch.cuda.synchronize()
        del part
    if int(status[0].item()):
        raise SystemExit("packing the device-generated scene raised a status bit")
    return PackedScene.from_packed_image(geo["positions"], geo["log_scales"], geo["quats"], geo["freq"], geo["att"], image, H,
                                         device=dev)


class Workload:
    """One named workload set up on this rank: scene, work units (view, band of tile rows), renderer."""

    def __init__(self, name, args, dev, world, rank, lib, timed_bcast=False, own_scene=False):
        import torch
        from mlp_splatting_b200 import _lib as L
        from mlp_splatting_b200 import sharding, synthetic as syn
        from mlp_splatting_b200.engine import FrameRenderer, PackedScene
        self.name, self.dev, self.world, self.rank, self.lib = name, dev, world, rank, lib
        cfg = self.cfg = dict(syn.WORKLOADS[name])
        for key, val in (("W", args.width), ("H", args.height), ("n", args.primitives)):
            if val:
                cfg[key] = int(val)       # a reduced copy of the workload (profiler captures)
        self.prec = L.PRECISION_F16 if args.precision == "fp16" else L.PRECISION_F32
        self.scene_np, self.bcast_s = None, 0.0
        if cfg.get("on_device"):
            if self.prec != L.PRECISION_F16:
                raise SystemExit(f"{name} is generated on the device and keeps only the fp16 weight image")
            self.ps = packed_scene_on_device(cfg, dev, lib)
        else:
            # own_scene: every rank draws the (seeded) scene itself instead of receiving it from rank 0, so that setting
            # the workload up involves no collective (the side measurements must not be able to desynchronise the ranks)
            if rank == 0 or own_scene:
                self.scene_np = syn.make_scene(cfg["n"], cfg["seed"], mu=cfg["mu"], hidden=cfg.get("hidden", 32),
                                               feat_dim=cfg.get("feat_dim", 0), pe_sigma=0.01 if args.encoder == "integrated" else 0.0)
            t_b0 = time.perf_counter()
            if own_scene:
                scene_t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in self.scene_np.items()
                           if isinstance(v, np.ndarray)}
            else:
                scene_t = sharding.broadcast_scene(self.scene_np, dev, src=0)
            torch.cuda.synchronize()
            self.bcast_s = time.perf_counter() - t_b0 if world > 1 else 0.0
            self.ps = PackedScene(*[scene_t[k] for k in ("positions", "log_scales", "quats") + WK], scene_t["freq"], scene_t["att"],
                                  feat_attr=scene_t.get("feat_attr"), device=dev, pack_f16=(self.prec == L.PRECISION_F16))
        # Work units of this rank.  Single-view workloads: one view per rank on the circle of radius 3 (weak
        # scaling, per-GPU work fixed).  Multi-view workloads: the workload's views are shared between the
        # ranks, by view and then by band of tile rows (strong scaling, total work fixed).
        self.nviews = int(cfg["views"])
        nty = (cfg["H"] + 7) // 8
        self.want_feat = cfg.get("feat_dim", 0) > 0
        if self.nviews == 1:
            # face-on views only (0/90/180/270 degrees): seen along a diagonal the same cube puts more than
            # 1,536 candidates into some tiles, which the path rejects exactly as the reference does
            self.units = [(syn.make_camera(cfg["W"], cfg["H"], azimuth_deg=90.0 * (rank % 4)), None)]
            self.frames_per_step, self.scaling = world, "weak"
        else:
            self.units = [(syn.make_camera(cfg["W"], cfg["H"], azimuth_deg=360.0 * v / self.nviews), (r0, r1) if (r0, r1) != (0, nty) else None)
                          for v, r0, r1 in sharding.assign(self.nviews, nty, world, rank)]
            self.frames_per_step, self.scaling = self.nviews, "strong"
        self.cam = self.units[0][0] if self.units else syn.make_camera(cfg["W"], cfg["H"])
        self.r = FrameRenderer(cfg["W"], cfg["H"], device=dev)
        self.batches, self.view_batch = [], int(getattr(args, "view_batch", 16))
        self.dev_rays = []
        for c, _rows in self.units:
            rd_dev = torch.from_numpy(c["rays_d"]).to(dev)
            rd_u = torch.empty_like(rd_dev)
            L.check(lib.mlpsp_normalize_rows(L.ptr(rd_dev), L.ptr(rd_u), self.r.P, 3, None), "normalize")
            self.dev_rays.append((torch.from_numpy(c["rays_o"]).to(dev), rd_u))
        # the step after the feature map, for workloads that name a decoder: decoder + text query in one kernel
        self.dec = self.text = self.labels = None
        if cfg.get("decoder"):
            from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder
            dc = cfg["decoder"]
            dw, dtext = syn.make_decoder(cfg["feat_dim"], dc["hidden"], dc["out_dim"], dc["classes"], seed=dc["seed"])
            self.dec = FeatureUpsampleDecoder(cfg["feat_dim"], dc["out_dim"], dc["hidden"], device=dev)
            self.dec.load_state_dict({k: torch.from_numpy(v) for k, v in dw.items()})
            self.text = torch.from_numpy(dtext).to(dev)
        self.score_dim = 0
        if cfg.get("text_query"):
            tq = cfg["text_query"]
            qtext = torch.from_numpy(np.random.default_rng(tq["seed"]).normal(size=(tq["classes"], cfg["feat_dim"])).astype(np.float32))
            self.ps = self.ps.with_text_query(qtext)
            self.score_dim = tq["classes"]

    def make_batches(self, per_view):
        """Multi-view workloads whose units are whole views render them in batches (mlpsp_render_frames): one
        evaluator launch per wave serves every view of a batch, so a primitive's weights are fetched once per wave
        instead of once per wave and view.  per_view = [(pairs, records)] of the views rendered alone (sizing)."""
        from mlp_splatting_b200.engine import ViewBatchRenderer
        self.batches = []
        cap = self.view_batch
        if cap < 2 or self.nviews == 1 or self.want_feat or len(self.units) < 2 or any(rows is not None for _c, rows in self.units):
            return
        for b0 in range(0, len(self.units), cap):
            idx = list(range(b0, min(b0 + cap, len(self.units))))
            pairs = int(1.25 * max(per_view[i][0] for i in idx)) + 4096
            records = int(1.1 * sum(per_view[i][1] for i in idx)) + 65536
            br = ViewBatchRenderer(self.cfg["W"], self.cfg["H"], len(idx), device=self.dev, max_pairs=pairs, max_records=records)
            self.batches.append((br, idx))

    def frame(self, check=False):
        cfg, r = self.cfg, self.r
        out = None
        if self.batches:
            for br, idx in self.batches:
                out = br.render(self.ps, [self.dev_rays[i][0] for i in idx], [self.dev_rays[i][1] for i in idx], THRESHOLD,
                                [self.units[i][0]["view"] for i in idx], [self.units[i][0]["proj"] for i in idx],
                                precision=self.prec, rays_normalized=True)[-1]
            return out
        for (c, rows), (ro_u, rd_u) in zip(self.units, self.dev_rays):
            out = r.render(self.ps, ro_u, rd_u, THRESHOLD, view=c["view"], proj=c["proj"], precision=self.prec,
                           rays_normalized=True, check=check, tile_rows=rows, want_feat=self.want_feat)
            if self.dec is not None:
                self.labels = self.dec.classify(r.feat.view(cfg["H"], cfg["W"], cfg["feat_dim"]), self.text, check=check)
            if self.score_dim:
                from mlp_splatting_b200.feature_decoder import score_labels
                self.labels = score_labels(r.feat.view(cfg["H"], cfg["W"], self.score_dim))
        return out

    def size_and_count(self):
        """Sizing pass (grows scratch if needed) and the per-step record totals of this rank."""
        self.frame(check=True)
        stats = self.r.last_stats
        if len(self.units) > 1:
            tot = dict(records=0, used=0, work_total=0, work_small=0)
            per_view = []
            for (c, rows), (ro_u, rd_u) in zip(self.units, self.dev_rays):
                self.r.render(self.ps, ro_u, rd_u, THRESHOLD, view=c["view"], proj=c["proj"], precision=self.prec,
                              rays_normalized=True, tile_rows=rows, want_feat=self.want_feat)
                for k in tot:
                    tot[k] += getattr(self.r.last_stats, k)
                per_view.append((self.r.last_stats.pairs, self.r.last_stats.records))
            self.make_batches(per_view)
            if self.batches:
                # the batches evaluate the same records in fewer, fuller work items
                self.frame()
                tot["work_total"] = sum(br.last_stats.work_total for br, _ in self.batches)
                tot["work_small"] = sum(br.last_stats.work_small for br, _ in self.batches)
                assert sum(br.last_stats.records for br, _ in self.batches) == tot["records"]
            stats.records, stats.used, stats.work_total, stats.work_small = tot["records"], tot["used"], tot["work_total"], tot["work_small"]
        self.stats = stats
        return stats


def barrier(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def timed_block(wl, flush, steps, world):
    """K frames, device time per frame by CUDA events, L2 flushed between frames; max over ranks of the summed time."""
    import torch
    import torch.distributed as dist
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier(world)
    wall0 = time.perf_counter()
    for a, b in evs:
        flush.fill_(1)
        a.record(); wl.frame(); b.record()
    barrier(world)
    wall = time.perf_counter() - wall0
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], dtype=torch.float64, device=wl.dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), wall


def class_times(wl, flush, steps):
    """Per-kernel-class device time (separate pass: event pairs around every launch group)."""
    import torch
    from mlp_splatting_b200 import _lib as L
    lib = wl.lib
    lib.mlpsp_timing_enable(1)
    per_class0 = (C.c_int64 * 8)()
    lib.mlpsp_kernel_launches(per_class0, 8)
    for _ in range(steps):
        flush.fill_(1); wl.frame()
    torch.cuda.synchronize()
    ms_cls = (C.c_float * 8)()
    L.check(lib.mlpsp_timing_collect(ms_cls, 8), "timing_collect")
    lib.mlpsp_timing_enable(0)
    per_class1 = (C.c_int64 * 8)()
    lib.mlpsp_kernel_launches(per_class1, 8)
    return {name: {"ms_per_step": ms_cls[i] / steps, "launches_per_step": (per_class1[i] - per_class0[i]) / steps}
            for i, name in enumerate(L.KERNEL_CLASSES)}


def evaluator_roofline(wl, classes, workload):
    pk = peaks()
    stats = wl.stats
    hidden = int(wl.cfg.get("hidden", 32))
    mlp_ms = classes["mlp"]["ms_per_step"]
    n_launch = max(classes["mlp"]["launches_per_step"], 1)
    flops_step = stats.records * flop_per_record(hidden)
    achieved_tf = flops_step / (mlp_ms / 1e3) / 1e12 if mlp_ms > 0 else 0.0
    roofline = {"kernel": "k_mlp_tc (per-primitive MLP, tcgen05)", "bound": "tensor", "achieved": achieved_tf,
                "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved_tf / pk["bf16_tflops"],
                "peak_source": pk["source"] + " burst", "traffic": None,
                "flop_per_launch": flops_step / n_launch, "avg_launch_ms": mlp_ms / n_launch,
                "share_of_step": mlp_ms / max(sum(c["ms_per_step"] for c in classes.values()), 1e-9)}
    # Algorithmic bytes of the evaluator: 32 B in + 16 B out per record, one weight image per work item.
    alg_bytes = stats.records * 48 + stats.work_total * weight_image_bytes(hidden)
    roofline["hbm_view"] = {"algorithmic_bytes_per_launch": alg_bytes / n_launch,
                            "achieved_gbs": alg_bytes / (mlp_ms / 1e3) / 1e9 if mlp_ms > 0 else 0.0,
                            "peak_gbs": pk["hbm_gbs"],
                            "frac": (alg_bytes / (mlp_ms / 1e3) / 1e9 / pk["hbm_gbs"]) if mlp_ms > 0 else 0.0}
    rec = ncu_figures(workload)
    if rec is not None:
        roofline["traffic"] = rec["dram_bytes_per_frame"] / n_launch
        roofline["traffic_unit"] = "bytes per launch: ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over a frame's evaluator launches"
        roofline["ncu_pipes_pct"] = dict(rec["pipes_pct"], source=rec["source"])
    return roofline


def short_measure(name, args, dev, world, rank, lib, flush, steps):
    """frames/s, ms per step and the evaluator's rate of another named workload (no end-to-end arm)."""
    import torch
    import torch.distributed as dist
    # no collective anywhere in here: a rank that fails must not leave the others waiting (the ranks' figures are
    # put together afterwards, combine_other_workloads)
    wl = Workload(name, args, dev, world, rank, lib, own_scene=True)
    stats = wl.size_and_count()
    for _ in range(3):
        flush.fill_(1); wl.frame()
    dev_ms, _wall = timed_block(wl, flush, steps, 1)
    classes = class_times(wl, flush, min(steps, 5))
    bits = int(wl.r.status.cpu()[0])
    for br, _idx in wl.batches:
        bits |= int(br.lead.status.cpu()[0])
    rec_t = [float(stats.records), float(stats.work_total), float(stats.work_small)]
    hidden = int(wl.cfg.get("hidden", 32))
    mlp_ms = classes["mlp"]["ms_per_step"]
    # what the evaluator must move on this rank: 32 B in + 16 B out per record, one weight image per work item.  With
    # few records per primitive the weight images dominate and this, not the tensor pipe, is the roof.
    alg_bytes = stats.records * 48.0 + stats.work_total * weight_image_bytes(hidden)
    pk = peaks()
    hbm = {"algorithmic_gb_this_rank": alg_bytes / 1e9,
           "achieved_gbs": alg_bytes / (mlp_ms / 1e3) / 1e9 if mlp_ms > 0 else 0.0,
           "peak_gbs": pk["hbm_gbs"],
           "flop_per_byte": stats.records * flop_per_record(hidden) / max(alg_bytes, 1.0)}
    hbm["frac"] = hbm["achieved_gbs"] / pk["hbm_gbs"]
    hbm["tflops_at_hbm_peak"] = hbm["flop_per_byte"] * pk["hbm_gbs"] / 1e3
    out = {"frames_per_sec": wl.frames_per_step * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps, "steps": steps,
           "local": {"dev_ms": dev_ms, "records": rec_t[0], "work_total": rec_t[1], "work_small": rec_t[2]},
           "scaling": wl.scaling, "views_per_step": wl.frames_per_step, "hidden": hidden,
           "views_per_call": [len(idx) for _br, idx in wl.batches] if wl.batches else 1,
           "evaluator_tflops_this_rank": stats.records * flop_per_record(hidden) / (mlp_ms / 1e3) / 1e12 if mlp_ms > 0 else 0.0,
           "evaluator_hbm_view": hbm,
           "records_per_step": float(rec_t[0]), "rows_per_evaluator_block": float(rec_t[0]) / max(float(rec_t[1]), 1.0),
           "fill_of_evaluator_blocks": float(rec_t[0]) / max(128.0 * float(rec_t[1] - rec_t[2]) + 32.0 * float(rec_t[2]), 1.0),
           "small_group_share_of_blocks": float(rec_t[2]) / max(float(rec_t[1]), 1.0),
           "kernel_classes_ms": {k: round(v["ms_per_step"], 4) for k, v in classes.items()},
           "status_bits": bits, "data": "generated on the device" if wl.cfg.get("on_device") else "generated on the host"}
    del wl
    torch.cuda.empty_cache()
    return out


def combine_other_workloads(per_rank):
    """Rank 0: one record per workload from the ranks' local ones (gathered objects).  The step time is the slowest
    rank's, the record counts are sums; a failure on any rank is reported instead of figures."""
    out = {}
    for name in per_rank[0]:
        recs = [pr.get(name) for pr in per_rank]
        if all(isinstance(r, dict) and "failed" not in r and "local" not in r for r in recs):
            out[name] = recs[0]          # a measurement of rank 0 alone
            continue
        failed = [f"rank {i}: {r.get('failed', 'missing') if isinstance(r, dict) else 'missing'}" for i, r in enumerate(recs)
                  if not isinstance(r, dict) or "failed" in r or "local" not in r]
        if failed:
            out[name] = {"failed": "; ".join(failed)[:600]}
            continue
        r0 = dict(recs[0])
        loc = [r.pop("local") if r is r0 else r["local"] for r in [r0] + recs[1:]]
        dev_ms = max(l["dev_ms"] for l in loc)
        rec, wt, ws = (sum(l[k] for l in loc) for k in ("records", "work_total", "work_small"))
        r0["frames_per_sec"] = r0["views_per_step"] * r0["steps"] / (dev_ms / 1e3)
        r0["ms_per_step"] = dev_ms / r0["steps"]
        r0["records_per_step"] = rec
        r0["rows_per_evaluator_block"] = rec / max(wt, 1.0)
        r0["fill_of_evaluator_blocks"] = rec / max(128.0 * (wt - ws) + 32.0 * ws, 1.0)
        r0["small_group_share_of_blocks"] = ws / max(wt, 1.0)
        r0["status_bits"] = 0
        for r in recs:
            r0["status_bits"] |= int(r["status_bits"])
        out[name] = r0
    return out


def weight_gradient_measure(dev, primitives=50000, per=100):
    """Per-primitive weight gradients (the backward side of the record path) on synthetic primitive-major records:
    ms per call of the IEEE FP32 kernel and of the tensor-core kernel with binary16 / bfloat16 operands."""
    import torch
    from mlp_splatting_b200.primitive_csr import PrimitiveCSR
    from mlp_splatting_b200.primitive_gemm import grouped_weight_gradients, prepare_groups
    g = torch.Generator().manual_seed(3)
    counts = torch.poisson(torch.full((primitives,), float(per)), generator=g).to(torch.int64)
    offsets = torch.cat((torch.zeros(1, dtype=torch.int64), counts.cumsum(0))).to(dev)
    R = int(offsets[-1])
    gd = torch.Generator(device=dev).manual_seed(4)
    x6 = torch.randn((R, 6), device=dev, generator=gd) * 0.2
    d3 = torch.randn((R, 4), device=dev, generator=gd)
    weights = [torch.randn((primitives, *shape), device=dev, generator=gd) * 0.1
               for shape in [(32, 72), (32,), (32, 32), (32,), (4, 32), (4,)]]
    freq = (2.0 ** torch.arange(6, dtype=torch.float32)).to(dev)
    att = torch.exp(-0.5 * freq.square() * 1e-4)
    csr = PrimitiveCSR(offsets, torch.arange(R, device=dev), x6, d3, None)
    groups = prepare_groups(csr, 512)
    out = {"primitives": primitives, "records": R, "segment_size": 512,
           "note": "ms per call through primitive_gemm.grouped_weight_gradients (host wrapper and flag read included)"}
    ref = None
    for name, dt in (("fp32_ms", torch.float32), ("f16_ms", torch.float16), ("bf16_ms", torch.bfloat16)):
        for _ in range(2):
            res = grouped_weight_gradients(csr, freq, att, weights, dtype=dt, groups=groups)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            res = grouped_weight_gradients(csr, freq, att, weights, dtype=dt, groups=groups)
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / 3
        if ref is None:
            ref = res[0]
        else:
            out[name.replace("_ms", "_rel_l2_dW1_vs_fp32")] = float((res[0] - ref).norm() / ref.norm())
    # 2 (mul, add) x 3 products (forward, adjoint, gradient) x the network's multiply-adds
    out["f16_tflops"] = R * 3 * 6912.0 / (out["f16_ms"] / 1e3) / 1e12
    del csr, groups, weights, x6, d3, res, ref
    torch.cuda.empty_cache()
    return out


def run_decoder(args):
    """The step after the feature map on its own: fused decoder + text query, decoder alone, full-width query."""
    import torch
    from mlp_splatting_b200 import synthetic as syn
    from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder, classify_feature_map
    dev = torch.device("cuda", 0)
    cin, hid, cout, ncls = 128, 128, 512, 20
    try:
        W, H = (int(v) for v in args.workload.split("_")[-1].split("x"))
    except ValueError:
        raise SystemExit("decoder workloads are named decoder_<width>x<height>")
    w, text = syn.make_decoder(cin, hid, cout, ncls, seed=1)
    dec = FeatureUpsampleDecoder(cin, cout, hid, device=dev)
    dec.load_state_dict({k: torch.from_numpy(v) for k, v in w.items()})
    x = torch.from_numpy(syn.make_feature_map(W, H, cin, seed=2)).to(dev)
    t = torch.from_numpy(text).to(dev)
    P = W * H

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    only = args.only
    flop = 2.0 * P * (cin * hid + 9 * hid * hid + hid * ncls)
    line = {"metric": "frames_per_sec", "unit": "frames/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"decoder_{cin}_{hid}_{cout}_c{ncls}_{W}x{H}",
                       "l2": f"input map {P * cin * 4 / 1e6:.0f} MB, decoded map {P * cout * 4 / 1e6:.0f} MB"}}
    if only in (None, "query"):
        ms_q = timed(lambda: dec.classify(x, t, check=False))
        line["fused_query"] = {"ms": ms_q, "algorithmic_tflops": flop / ms_q / 1e9, "bytes_per_pixel": 4 * cin + 8,
                               "gbs": P * (4 * cin + 8) / ms_q / 1e6}
        line.update(value=1e3 / ms_q, ms_per_step=ms_q)
    if only in (None, "decode", "full_width"):
        y = dec.decode_hwc(x)
    if only in (None, "decode"):
        ms_d = timed(lambda: dec.decode_hwc(x, check=False))
        line["decode"] = {"ms": ms_d, "bytes_per_pixel": 4 * (cin + cout), "gbs": P * 4 * (cin + cout) / ms_d / 1e6}
        line.setdefault("value", 1e3 / ms_d); line.setdefault("ms_per_step", ms_d)
    if only in (None, "full_width"):
        ms_f = timed(lambda: classify_feature_map(y, t))
        line["full_width_query"] = {"ms": ms_f, "bytes_per_pixel": 4 * cout + 8, "gbs": P * (4 * cout + 8) / ms_f / 1e6}
        line.setdefault("value", 1e3 / ms_f); line.setdefault("ms_per_step", ms_f)
    dec._check_status("bench")
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=HEADLINE)
    ap.add_argument("--other-workloads-multi", action="store_true",
                    help="also run the other workloads' short measurements when several ranks are used")
    ap.add_argument("--e2e-depth", type=int, default=8,
                    help="frames in flight in the end-to-end arm (measured on one B200: 2 -> 731, 3 -> 867, 4 -> 899, "
                         "6 -> 971, 8 -> 984, 12 -> 990 frames/s)")
    ap.add_argument("--view-batch", type=int, default=16,
                    help="views of a multi-view workload rendered per call (0 or 1: view by view, as the reference does)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="fp16", choices=["fp16", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="skip the short measurements of the other named workloads that the default run adds")
    ap.add_argument("--width", type=int, default=0, help="override the workload's image width (reduced captures)")
    ap.add_argument("--height", type=int, default=0, help="override the workload's image height")
    ap.add_argument("--primitives", type=int, default=0, help="override the workload's primitive count")
    ap.add_argument("--only", default=None, choices=["query", "decode", "full_width"],
                    help="decoder workloads: time one of the three steps only")
    ap.add_argument("--e2e-image", default="f32", choices=["f32", "f16"],
                    help="format of the image copied back to the host in the end-to-end arm")
    ap.add_argument("--encoder", default="integrated", choices=["integrated", "fourier"],
                    help="integrated: the reference default (bands attenuated by exp(-f^2 sigma^2 / 2), sigma 0.01); "
                         "fourier: unattenuated power-of-two bands")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if args.workload.startswith("decoder_"):
        return run_decoder(args)
    if args.workload == "weight_gradients":
        # the backward side of the record path alone: FP32 kernel beside the tensor-core kernel (one GPU)
        import torch
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        print(json.dumps(dict(metric="weight_gradient_ms", n_gpus=1, data="synthetic",
                              **weight_gradient_measure(dev, primitives=args.primitives or 50000))), flush=True)
        return

    import torch
    import torch.distributed as dist
    from mlp_splatting_b200 import _lib as L

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

    wl = Workload(args.workload, args, dev, world, rank, lib)
    cfg, r, ps, prec = wl.cfg, wl.r, wl.ps, wl.prec
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    stats = wl.size_and_count()
    for _ in range(args.warmup):
        flush.fill_(1); wl.frame()
    barrier(world)

    # ---- timed region: K frames; then further blocks of K frames until a second of device time has been seen ----
    clock_mark = sampler.mark()
    launches0 = lib.mlpsp_kernel_launches(None, 0)
    dev_ms_max, wall = timed_block(wl, flush, args.steps, world)
    launches = lib.mlpsp_kernel_launches(None, 0) - launches0
    clock_end = sampler.mark()
    blocks = [dev_ms_max / args.steps]
    spent = dev_ms_max
    while spent < 1000.0 and len(blocks) < 64:
        ms, _w = timed_block(wl, flush, args.steps, world)
        blocks.append(ms / args.steps)
        spent += ms
    # nvidia-smi answers every 20-100 ms and the first block may be shorter than that: the window that opened with the
    # timed region is read once it holds a handful of samples (the repeated blocks are the same frames)
    t_c = time.perf_counter()
    while rank == 0 and sampler.proc is not None and sampler.mark() - clock_mark < 5 and time.perf_counter() - t_c < 1.5:
        wl.frame(); torch.cuda.synchronize()
    clocks = None
    if rank == 0:
        clocks = sampler.summary(clock_mark)
        clocks["window"] = (f"the timed block of {args.steps} steps and the {len(blocks) - 1} repeated blocks after it "
                            f"({sampler.mark() - clock_mark} samples; {max(clock_end - clock_mark, 0)} of them inside the first block)")
    barrier(world)
    bits = int(r.status.cpu()[0])
    if bits & ~L.BIT_NUMERIC:
        raise SystemExit(f"render status bits {bits} during the timed region")
    ms_per_step = dev_ms_max / args.steps
    fps = wl.frames_per_step * args.steps / (dev_ms_max / 1e3)
    rec_t = torch.tensor([float(stats.records), float(stats.used)], dtype=torch.float64, device=dev)
    if world > 1 and wl.nviews > 1:
        dist.all_reduce(rec_t)   # records of the whole step (all views), summed over ranks

    classes = class_times(wl, flush, min(args.steps, 10))
    roofline = evaluator_roofline(wl, classes, args.workload if (prec == L.PRECISION_F16 and args.encoder == "integrated") else "")

    # ---- end to end: pinned host rays in, image out, status checked, through the public host API.
    # Several frames are kept in flight (FramePipeline, --e2e-depth): every step still copies its own rays to the
    # device and its own image back inside the timed region; the copies and the part-filled kernels of one frame
    # overlap those of the others.
    # A pinhole camera has one ray origin: it travels as a [1,3] tensor and is expanded on the device.
    from mlp_splatting_b200.engine import FramePipeline
    depth = max(1, int(args.e2e_depth))
    pipe = FramePipeline(ps, cfg["W"], cfg["H"], depth=depth, max_records=r.max_records)
    img_dtype = torch.float16 if args.e2e_image == "f16" else torch.float32
    outs = [(torch.empty((r.P, 3), dtype=img_dtype).pin_memory(), torch.empty((r.P, 1), dtype=img_dtype).pin_memory())
            for _ in range(depth)]
    host_rays = []
    for c, _rows in wl.units:
        one_origin = bool((c["rays_o"] == c["rays_o"][:1]).all())
        ro = torch.from_numpy(np.ascontiguousarray(c["rays_o"][:1] if one_origin else c["rays_o"])).pin_memory()
        host_rays.append((ro, torch.from_numpy(c["rays_d"]).pin_memory()))

    def e2e_run(k):
        j = 0
        for _i in range(k):
            for (c, rows), (roh, rdh) in zip(wl.units, host_rays):
                o = outs[j % depth]; j += 1
                pipe.submit(roh, rdh, THRESHOLD, c["view"], c["proj"], out_rgb_host=o[0], out_alpha_host=o[1],
                            precision=prec, tile_rows=rows)
        pipe.drain()

    e2e_run(2 * depth)

    def e2e_block():
        """One block of K steps through the pipeline, filled and drained: wall seconds, max over ranks."""
        barrier(world)
        e0 = time.perf_counter()
        e2e_run(args.steps)
        barrier(world)
        e_t = torch.tensor([time.perf_counter() - e0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(e_t, op=dist.ReduceOp.MAX)
        return float(e_t.item())

    # the block is short (K frames of about a millisecond), so it is repeated for about half a second and the median
    # block is reported; every block pays for filling and draining the pipeline
    e2e_blocks = [e2e_block()]
    while sum(e2e_blocks) < 0.5 and len(e2e_blocks) < 200:
        e2e_blocks.append(e2e_block())
    e2e_fps = wl.frames_per_step * args.steps / statistics.median(e2e_blocks)
    e2e_first = wl.frames_per_step * args.steps / e2e_blocks[0]
    nunits = max(len(wl.units), 1)
    last = (args.steps * nunits - 1) % depth
    e2e_err = float((outs[last][0].to(dev).float() - r.rgb).abs().max()) if wl.units else 0.0   # must reproduce the resident-input frame
    h2d = sum(int(a.numel() + b.numel()) * 4 for a, b in host_rays)
    d2h = nunits * (r.P * 4 * img_dtype.itemsize + 64)

    # Two side measurements that explain the end-to-end figure when several GPUs share one host:
    #  * the same arm with a binary16 host image (the pipeline converts on the device; FP32 stays the default
    #    because it is what the reference returns);
    #  * the step's copies alone (rays in, image out, no rendering) from every rank at once: what the host's
    #    PCIe side delivers for this traffic, i.e. the ceiling of the arm above on this machine.
    e2e_extra = {}
    if args.e2e_image == "f32" and wl.units:
        outs16 = [(torch.empty((r.P, 3), dtype=torch.float16).pin_memory(), torch.empty((r.P, 1), dtype=torch.float16).pin_memory())
                  for _ in range(depth)]
        outs_f32, outs = outs, outs16
        e2e_run(2 * depth)
        b16 = [e2e_block()]
        while sum(b16) < 0.3 and len(b16) < 100:
            b16.append(e2e_block())
        outs = outs_f32
        e2e_extra["f16_image"] = {"value": wl.frames_per_step * args.steps / statistics.median(b16),
                                  "d2h_bytes_per_step": nunits * (r.P * 4 * 2 + 64)}
        del outs16
    if wl.units:
        dsrc = [(torch.empty((r.P, 3), device=dev), torch.empty((r.P, 3), device=dev), torch.empty((r.P, 1), device=dev)) for _ in range(3)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

        def copies_block():
            barrier(world)
            c0 = time.perf_counter()
            j = 0
            for _i in range(args.steps):
                for (_roh, rdh) in host_rays:
                    k = j % 3; j += 1
                    with torch.cuda.stream(s_in):
                        dsrc[k][0].copy_(rdh, non_blocking=True)
                    with torch.cuda.stream(s_out):
                        outs[k % depth][0].copy_(dsrc[k][1], non_blocking=True)
                        outs[k % depth][1].copy_(dsrc[k][2], non_blocking=True)
            torch.cuda.synchronize()
            barrier(world)
            c_t = torch.tensor([time.perf_counter() - c0], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(c_t, op=dist.ReduceOp.MAX)
            return float(c_t.item())

        copies_block()
        cb = [copies_block()]
        while sum(cb) < 0.3 and len(cb) < 100:
            cb.append(copies_block())
        fps_c = wl.frames_per_step * args.steps / statistics.median(cb)
        e2e_extra["copies_only"] = {"value": fps_c, "unit": "frames/s",
                                    "gbs_both_directions": fps_c * (h2d + d2h) / max(nunits, 1) / 1e9,
                                    "note": "the step's host-to-device and device-to-host copies alone, all ranks at once"}
        del dsrc

    others = None
    reduced = bool(args.width or args.height or args.primitives)
    # The side measurements run on one GPU by default.  With several ranks they are opt-in (--other-workloads-multi):
    # they add minutes of work in which any rank-local failure could cost the whole line, and the headline figures of
    # a scaling run do not need them.
    if (args.workload == HEADLINE and not args.no_other_workloads and prec == L.PRECISION_F16 and not reduced
            and (world == 1 or args.other_workloads_multi)):
        del pipe
        others = {}
        for name in OTHER_WORKLOADS:
            from mlp_splatting_b200 import synthetic as syn
            views = int(syn.WORKLOADS[name]["views"])
            if world > 1 and views == 1:
                continue          # single-view workloads scale like the headline one
            try:
                others[name] = short_measure(name, args, dev, world, rank, lib, flush, steps=5 if views < 8 else 2)
            except Exception as exc:     # the headline line must not be lost over an extra measurement
                others[name] = {"failed": f"{type(exc).__name__}: {exc}"[:300]}
        if world == 1:
            try:
                others["weight_gradients_50k_x100"] = weight_gradient_measure(dev)
            except Exception as exc:
                others["weight_gradients_50k_x100"] = {"failed": f"{type(exc).__name__}: {exc}"[:300]}
        # the one collective of the side measurements: every rank reaches it, whatever happened above
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, others)
            others = combine_other_workloads(gathered) if rank == 0 else None
        else:
            others = combine_other_workloads([others])

    if rank == 0:
        line = {
            "metric": "frames_per_sec", "value": fps, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": wl.scaling,
            "vs_baseline": None, "dtype": "f16" if prec == L.PRECISION_F16 else "f32", "data": "synthetic",
            "config": workload_config(args.workload, cfg, world, args.encoder),
            "repeat": {"blocks": len(blocks), "steps_per_block": args.steps, "ms_per_step_median": statistics.median(blocks),
                       "ms_per_step_min": min(blocks), "ms_per_step_max": max(blocks),
                       "note": "value and ms_per_step are the first block; the others repeat it until 1 s of device time"},
            "record_mlp_evals_per_sec": float(rec_t[0]) * (fps / wl.frames_per_step if wl.nviews > 1 else fps),
            "records_per_frame": {"evaluated": stats.records, "composited": stats.used, "candidate_pairs": stats.pairs, "pairs_after_tile_pretest": stats.pairs_kept, "evaluator_blocks": stats.work_total,
                                  "small_group_blocks": stats.work_small,
                                  "rows_per_evaluator_block": stats.records / max(stats.work_total, 1),
                                  "fill_of_evaluator_blocks": stats.records / max(128 * (stats.work_total - stats.work_small) + 32 * stats.work_small, 1),
                                  "waves": stats.waves, "max_tile_len": stats.max_tile_len},
            "e2e": {"value": e2e_fps, "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "frames_in_flight": depth, "image": args.e2e_image, "max_abs_diff_vs_resident_frame": e2e_err,
                    "blocks": len(e2e_blocks), "first_block": e2e_first, **e2e_extra,
                    "fastest_block": wl.frames_per_step * args.steps / min(e2e_blocks),
                    "slowest_block": wl.frames_per_step * args.steps / max(e2e_blocks),
                    "note": "median of the repeated K-step blocks (each filled and drained); frames in flight overlap and L2 is "
                            "not flushed between them, so this can exceed `value`, which times one frame at a time with "
                            "L2 flushed; a single ray origin travels as [1,3]"},
            "gpu_launches": int(launches),
            "kernel_classes": classes,
            "roofline": roofline,
            "clocks": clocks,
            "scene_broadcast_s": wl.bcast_s,
            "wall_ms_per_step": wall * 1e3 / args.steps,
        }
        if others is not None:
            line["other_workloads"] = others
        if not args.no_cpu_baseline and world == 1 and wl.scene_np is not None:
            cb = cpu_baseline(wl.scene_np, wl.cam, budget_s=15.0)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    sampler.stop()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
