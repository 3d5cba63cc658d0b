"""Launch-shape sweep for the streaming decode kernel on the GPU at hand.

    python -m fastforwardattention_b200.tune --workload long-8192 [--out sweep.json]

Times the one-pass kernel over a grid of (tile_rows, stages, consumer_warps, ctas_per_sm) on
one engine instance and prints the shapes ranked by achieved HBM bandwidth.  The winners are
what the measured planner table in csrc/ffa_c_api.cu is filled from.  This replaces the
reference's fitted cost model (kernel_launch_utils.h:85-132) with direct measurement.
"""
from __future__ import annotations

import argparse
import itertools
import json

import torch

from .workloads import CONFIGS, device_prompt_kv


def time_shape(engines, w, q, k, v, out, shape, steps):
    """Median over 3 replays of a CUDA graph holding `steps` back-to-back launches that rotate
    over the engine replicas (together larger than L2, so every launch streams from HBM and
    no flush kernel perturbs the timing).  Returns ms per launch."""
    for e in engines:
        e.set_launch(*shape)
    got = engines[0].launch_shape(w.max_len - 1)
    if (got["tile_rows"], got["stages"], got["consumer_warps"], got["ctas_per_sm"]) != tuple(shape):
        return None, got   # did not fit in shared memory as asked
    t = w.max_len - 1
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(len(engines)):
            engines[i].attention(q, k, v, w.scale, t, 0.0, out=out)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(steps):
            engines[i % len(engines)].attention(q, k, v, w.scale, t, 0.0, out=out)
    ms = []
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b) / steps)
    ms.sort()
    return ms[1], got


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="long-8192", choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--tile-rows", default="16,32,64,128")
    ap.add_argument("--stages", default="2,3,4")
    ap.add_argument("--warps", default="2,4,8")
    ap.add_argument("--cps", default="1,2,4")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (per-GPU shard sizes)")
    ap.add_argument("--top", type=int, default=12)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from dataclasses import replace

    from . import FastForwardAttn

    w = CONFIGS[args.workload]
    if args.heads:
        w = replace(w, H=args.heads)
    dev = torch.device("cuda:0")
    es = w.dtype.itemsize
    alg = es * w.B * w.H * w.Dh * (2 * (w.max_len - 1) + 6)
    nrep = max(1, min(16, -(-int(600e6) // alg)))      # replicas: together well beyond the 126 MB L2
    engines = []
    for r in range(nrep):
        K, V = device_prompt_kv(replace(w, seed=w.seed + r), dev)
        e = FastForwardAttn(K, V, w.max_len, False)
        del K, V
        kc, vc = e.get_cache()                          # rows the decode steps would have appended
        kc[:, :, w.prompt:].normal_()
        vc[:, :, w.prompt:].normal_()
        engines.append(e)
    q, k, v = (torch.randn(w.B, w.H, 1, w.Dh, device=dev).to(w.dtype) for _ in range(3))
    out = torch.empty(w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
    rows = []
    ints = lambda s: [int(x) for x in s.split(",")]
    for shape in itertools.product(ints(args.tile_rows), ints(args.stages), ints(args.warps), ints(args.cps)):
        ms, got = time_shape(engines, w, q, k, v, out, shape, max(args.steps, nrep))
        if ms is None:
            continue
        rows.append({"tile_rows": shape[0], "stages": shape[1], "warps": shape[2], "cps": shape[3], "us": ms * 1e3,
                     "gbs": alg / ms / 1e6, "grid": got["grid"], "smem": got["smem_bytes"]})
    assert all(e.device_status() == 0 for e in engines)
    for e in engines:
        e.set_launch()
    ms, got = time_shape(engines, w, q, k, v, out, (got_default := engines[0].launch_shape(w.max_len - 1))["tile_rows"] and
                         (got_default["tile_rows"], got_default["stages"], got_default["consumer_warps"], got_default["ctas_per_sm"]),
                         max(args.steps, nrep))
    rows.sort(key=lambda r: r["us"])
    print(json.dumps({"workload": w.name, "heads": w.H, "alg_MB": alg / 1e6, "replicas": nrep,
                      "planner_choice": got, "planner_us": ms * 1e3, "planner_gbs": alg / ms / 1e6}))
    for r in rows[:args.top]:
        print(json.dumps(r))
    print("worst:", json.dumps(rows[-1]))
    if args.out:
        json.dump({"workload": w.name, "heads": w.H, "alg_bytes": alg, "rows": rows}, open(args.out, "w"))


if __name__ == "__main__":
    main()
