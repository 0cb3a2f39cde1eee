"""Timing of the feature decoder and text query on one GPU (synthetic weights and maps).

    python mlp-splatting_b200/decoder_bench.py [--width 1200 --height 680 --in-dim 128 --hidden 128 --out-dim 512
                                                --classes 20 --steps 20 --warmup 3]

Prints one JSON line: milliseconds per frame of the fused query (decoder + text arg-max in one kernel), of the
decoder alone (decoded map written) and of the full-width text query, timed with CUDA events on the launching
stream; the input map (and for the full-width query the decoded map) is larger than L2 at the default size.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mlp_splatting_b200 import synthetic as syn                                   # noqa: E402
from mlp_splatting_b200.feature_decoder import FeatureUpsampleDecoder, classify_feature_map   # noqa: E402


def timed(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--width", type=int, default=1200)
    ap.add_argument("--height", type=int, default=680)
    ap.add_argument("--in-dim", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--out-dim", type=int, default=512)
    ap.add_argument("--classes", type=int, default=20)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", choices=["query", "decode", "full_width"], default=None)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    w, text = syn.make_decoder(a.in_dim, a.hidden, a.out_dim, a.classes, seed=1)
    dec = FeatureUpsampleDecoder(a.in_dim, a.out_dim, a.hidden, device=dev)
    dec.load_state_dict({k: torch.from_numpy(v) for k, v in w.items()})
    x = torch.from_numpy(syn.make_feature_map(a.width, a.height, a.in_dim, seed=2)).to(dev)
    t = torch.from_numpy(text).to(dev)
    P = a.width * a.height
    out = {"workload": f"decoder_{a.in_dim}_{a.hidden}_{a.out_dim}_c{a.classes}_{a.width}x{a.height}", "pixels": P}
    if a.only in (None, "query"):
        ms = timed(lambda: dec.classify(x, t, check=False), a.steps, a.warmup)
        flop = 2.0 * P * (a.in_dim * a.hidden + 9 * a.hidden * a.hidden + a.hidden * a.classes)
        out["fused_query"] = {"ms": ms, "algorithmic_tflops": flop / ms / 1e9,
                              "bytes_per_pixel": 4 * a.in_dim + 8, "gbs": P * (4 * a.in_dim + 8) / ms / 1e6}
    if a.only in (None, "decode", "full_width"):
        y = dec.decode_hwc(x)
    if a.only in (None, "decode"):
        ms = timed(lambda: dec.decode_hwc(x, check=False), a.steps, a.warmup)
        out["decode"] = {"ms": ms, "bytes_per_pixel": 4 * (a.in_dim + a.out_dim),
                         "gbs": P * 4 * (a.in_dim + a.out_dim) / ms / 1e6}
    if a.only in (None, "full_width"):
        ms = timed(lambda: classify_feature_map(y, t), a.steps, a.warmup)
        out["full_width_query"] = {"ms": ms, "bytes_per_pixel": 4 * a.out_dim + 8,
                                   "gbs": P * (4 * a.out_dim + 8) / ms / 1e6}
    dec._check_status("decoder_bench")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
