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


def time_shape(ffa, w, q, k, v, out, shape, steps, flush):
    ffa.set_launch(*shape)
    got = ffa.launch_shape(w.max_len - 1)
    if (got["tile_rows"], got["stages"], got["consumer_warps"], got["ctas_per_sm"]) != tuple(shape):
        return None, got   # did not fit in shared memory as asked
    t = w.max_len - 1
    for _ in range(3):
        ffa.attention(q, k, v, w.scale, t, 0.0, out=out)
    torch.cuda.synchronize()
    ms = []
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ffa.attention(q, k, v, w.scale, t, 0.0, out=out)
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b))
    ms.sort()
    return ms[len(ms) // 2], got


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="long-8192", choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=9)
    ap.add_argument("--tile-rows", default="16,32,64,128")
    ap.add_argument("--stages", default="2,3,4,6,8")
    ap.add_argument("--warps", default="4,8,12,16")
    ap.add_argument("--cps", default="1,2,3,4")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (per-GPU shard sizes)")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from . import FastForwardAttn
    from dataclasses import replace

    w = CONFIGS[args.workload]
    if args.heads:
        w = replace(w, H=args.heads)
    dev = torch.device("cuda:0")
    K, V = device_prompt_kv(w, dev)
    ffa = FastForwardAttn(K, V, w.max_len, False)
    del K, V
    # fill the rows the decode steps would have appended, so that t = max_len - 1 reads real data
    kc, vc = ffa.get_cache()
    kc[:, :, w.prompt:].normal_()
    vc[:, :, w.prompt:].normal_()
    q, k, v = (torch.randn(w.B, w.H, 1, w.Dh, device=dev).to(w.dtype) for _ in range(3))
    out = torch.empty(w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
    es = w.dtype.itemsize
    alg = es * w.B * w.H * w.Dh * (2 * (w.max_len - 1) + 6)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if alg < 4 * 126e6 else None
    rows = []
    ints = lambda s: [int(x) for x in s.split(",")]
    for shape in itertools.product(ints(args.tile_rows), ints(args.stages), ints(args.warps), ints(args.cps)):
        ms, got = time_shape(ffa, w, q, k, v, out, shape, args.steps, flush)
        if ms is None:
            continue
        rows.append({"tile_rows": shape[0], "stages": shape[1], "warps": shape[2], "cps": shape[3], "ms": ms,
                     "gbs": alg / ms / 1e6, "grid": got["grid"], "smem": got["smem_bytes"]})
    assert ffa.device_status() == 0
    rows.sort(key=lambda r: r["ms"])
    for r in rows[:25]:
        print(json.dumps(r))
    print("worst:", json.dumps(rows[-1]))
    if args.out:
        json.dump({"workload": w.name, "heads": w.H, "alg_bytes": alg, "rows": rows}, open(args.out, "w"))


if __name__ == "__main__":
    main()
