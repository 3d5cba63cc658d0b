"""Decode-attention benchmark: steps/s and achieved HBM bandwidth on 1/2/4/8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload long-32768] [--impl reference]

A "step" is one decode step of masked multi-head attention over the whole batch: append the
new k/v row, attend over rows 0..t, write out [B, H, Dh].  The default workload is the long
sequence configuration (bf16, batch 32, 32 heads, head_dim 128, final length 32768: prompt
32640 + 128 steps) on synthetic N(0,1) tensors.  With N > 1 (one process per GPU, torchrun)
the heads are sharded: every rank owns H/N heads and their KV shard; total work is fixed.

Prints ONE JSON line (rank 0): `value` = whole-job steps/s with inputs resident in HBM,
`e2e` = the same through the Python class with q/k/v in pinned host memory and the output
read back every step (plus the output all-gather when N > 1), `roofline` = algorithmic HBM
bytes per kernel launch over its CUDA-event duration against the measured copy bandwidth,
`cpu_baseline` = the reference's torch function timed on the host cores over a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from fastforwardattention_b200.workloads import CONFIGS, device_prompt_kv  # noqa: E402

METRIC = "decode_attention_steps_per_sec"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the streaming kernel divided by
# the launch's algorithmic bytes, from the ncu capture summarised under profiles/ (captured on
# the 2048-token case and scaled by bytes streamed, which is what the kernel's traffic is
# proportional to).
TRAFFIC_RATIO = 1.004


def algorithmic_bytes(es, B, H, Dh, t):
    """K and V rows 0..t-1 read once, q/k/v read, rows t written, out written."""
    return es * B * H * Dh * (2 * t + 6)


def gpu_id(dev):
    """nvidia-smi numbers physical GPUs; torch numbers visible ones.  The UUID names the same GPU in both."""
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        return str(dev.index or 0)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region (read-only query)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None   # an nvidia-smi id: index or GPU-<uuid>

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.rows = []
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 7:
                self.rows.append(f)

    def summary(self):
        if not getattr(self, "rows", None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.rows[0][1]),
                "power_w_max": max(float(r[2]) for r in self.rows), "reasons": reasons, "samples": len(self.rows)}


class CpuReferenceSample:
    """The reference's torch function (example.py:6-7) on the host cores over a bounded sample
    of the workload: `pairs` (batch, head) pairs of the full configuration at its final
    length.  One call of step() is one evaluation over the sample; the full-workload step
    time is extrapolated by the pair count ((batch, head) pairs are independent)."""

    def __init__(self, w, pairs=32):
        from oracle.ffa_oracle import torch_attn_func

        self.fn, self.w = torch_attn_func, w
        torch.set_num_threads(os.cpu_count() or 1)
        self.N, self.L = w.B * w.H, w.max_len
        self.pairs = min(self.N, pairs)
        g = torch.Generator().manual_seed(w.seed)
        self.K = torch.randn(self.pairs, self.L, w.Dh, generator=g).to(w.dtype)
        self.V = torch.randn(self.pairs, self.L, w.Dh, generator=g).to(w.dtype)
        self.q = torch.randn(self.pairs, 1, w.Dh, generator=g).to(w.dtype)
        self.cores = torch.get_num_threads()

    def step(self):
        t0 = time.perf_counter()
        self.fn(self.q, self.K, self.V, self.w.scale)
        return time.perf_counter() - t0

    def describe(self, n):
        return (f"{self.pairs} of {self.N} (batch, head) pairs at length {self.L}, {n} timed evaluations, "
                f"torch {str(self.w.dtype).split('.')[-1]} on CPU, extrapolated by pair count")

    def run(self, steps, warmup):
        for _ in range(warmup):
            self.step()
        dt = [self.step() for _ in range(steps)]
        full_step_s = statistics.mean(dt) * (self.N / self.pairs)
        return 1.0 / full_step_s


def run_reference(args, w):
    """Reference arm: the reference's own CPU statement of the path (its torch function; the
    reference has no other CPU implementation), all host threads, bounded sample per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    smp = CpuReferenceSample(w)
    probe = smp.step()
    steps = max(1, min(args.steps, int(120.0 / max(probe, 1e-3))))   # keep the arm within minutes
    value = smp.run(steps, min(args.warmup, 3))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "steps/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": 1e3 / value, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": str(w.dtype).split(".")[-1], "data": "synthetic",
            "config": workload_config(w, args.gpus),
            "cpu_baseline": {"value": value, "unit": "steps/s", "cores": smp.cores, "kind": "port",
                             "sample": smp.describe(steps)},
            "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(w, n):
    return {"workload": w.name, "batch": w.B, "heads": w.H, "head_dim": w.Dh, "prompt": w.prompt,
            "decode_steps": w.steps, "final_len": w.max_len, "p": w.p,
            "parallelism": f"heads sharded over {n} GPU(s), {w.H // n} heads each" if n > 1 else "single GPU",
            "l2": "inputs larger than L2: every step streams the whole KV cache shard from HBM"
                  if 2 * w.B * (w.H // n) * w.max_len * w.Dh * w.dtype.itemsize > 2 * 126e6 else
                  "KV shard smaller than L2; an L2 flush (256 MB write) runs between timed steps"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="long-32768", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--launch", default="", help="tile_rows,stages,consumer_warps,ctas_per_sm override (tuning)")
    args = ap.parse_args()
    full = CONFIGS[args.workload]
    if args.impl == "reference":
        return run_reference(args, full)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    import torch.distributed as dist

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from fastforwardattention_b200 import FastForwardAttn, ShardedFastForwardAttn, launch_count

    w = full.shard(rank, world) if world > 1 else full
    es = w.dtype.itemsize
    K, V = device_prompt_kv(w, dev)
    eng = ShardedFastForwardAttn(K, V, w.max_len, False) if world > 1 else None
    ffa = eng.engine if eng is not None else FastForwardAttn(K, V, w.max_len, False)
    del K, V
    torch.cuda.empty_cache()
    if args.launch:
        ffa.set_launch(*[int(x) for x in args.launch.split(",")])
    shape = ffa.launch_shape(w.max_len - 1)

    total = args.warmup + args.steps
    g = torch.Generator(device=dev).manual_seed(w.seed + 1)
    qkv_d = torch.randn(total, 3, w.B, w.H, 1, w.Dh, generator=g, device=dev, dtype=torch.float32).to(w.dtype)
    qkv_h = qkv_d.cpu().pin_memory()
    out_d = torch.empty(w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
    out_h = torch.empty(w.B, w.H, w.Dh, dtype=w.dtype).pin_memory()
    stage = torch.empty(3, w.B, w.H, 1, w.Dh, dtype=w.dtype, device=dev)
    small = 2 * w.B * w.H * w.max_len * w.Dh * es <= 2 * 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None
    t_of = lambda s: w.prompt + (s % w.steps)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- leg 1: inputs resident in HBM; per-launch events give the kernel's own duration ----
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for s in range(args.warmup):
        ffa.attention(qkv_d[s, 0], qkv_d[s, 1], qkv_d[s, 2], w.scale, t_of(s), 0.0, out=out_d)
    barrier()
    launches0 = launch_count()
    with ClockSampler(gpu_id(dev)) as clocks:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.steps):
            s = args.warmup + i
            if flush is not None:
                flush.zero_()
            ev[i][0].record()
            ffa.attention(qkv_d[s, 0], qkv_d[s, 1], qkv_d[s, 2], w.scale, t_of(s), 0.0, out=out_d)
            ev[i][1].record()
        stop.record()
        barrier()
    launches = launch_count() - launches0
    kernel_ms = [a.elapsed_time(b) for a, b in ev]
    loop_ms = sum(kernel_ms) if flush is not None else start.elapsed_time(stop)
    alg = [algorithmic_bytes(es, w.B, w.H, w.Dh, t_of(args.warmup + i)) for i in range(args.steps)]

    # ---- leg 2: end to end through the Python class with host buffers ----
    for s in range(min(3, args.warmup)):
        stage.copy_(qkv_h[s], non_blocking=True)
        o = (eng.attention(stage[0], stage[1], stage[2], w.scale, t_of(s), 0.0, gather=True) if eng is not None
             else ffa.attention(stage[0], stage[1], stage[2], w.scale, t_of(s), 0.0))
        out_h_full = torch.empty(o.shape, dtype=o.dtype).pin_memory()
        out_h_full.copy_(o, non_blocking=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        s = args.warmup + i
        stage.copy_(qkv_h[s], non_blocking=True)
        o = (eng.attention(stage[0], stage[1], stage[2], w.scale, t_of(s), 0.0, gather=True) if eng is not None
             else ffa.attention(stage[0], stage[1], stage[2], w.scale, t_of(s), 0.0))
        out_h_full.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the caller consumes the result every step
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    status = ffa.device_status()

    # ---- max over ranks ----
    times = torch.tensor([loop_ms, e2e_ms, sum(kernel_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    loop_ms, e2e_ms, ksum_ms = times.tolist()

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = sum(alg) / (ksum_ms * 1e-3) / 1e9          # per GPU: this rank's bytes over its kernel time
        per_launch_alg = sum(alg) / len(alg)
        line = {"metric": METRIC, "value": args.steps / (loop_ms * 1e-3), "unit": "steps/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": loop_ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": str(w.dtype).split(".")[-1], "data": "synthetic", "config": workload_config(full, world),
                "hbm_gbs_all_gpus": world * sum(alg) / (loop_ms * 1e-3) / 1e9,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": achieved / 8000.0,
                             "kernel": "ffa_stream_kernel (one-pass)", "bytes_per_launch": per_launch_alg,
                             "avg_launch_ms": ksum_ms / args.steps,
                             "traffic": TRAFFIC_RATIO * per_launch_alg if TRAFFIC_RATIO else None},
                "e2e": {"value": args.steps / (e2e_ms * 1e-3), "unit": "steps/s",
                        "h2d_bytes_per_step": 3 * w.B * w.H * w.Dh * es, "d2h_bytes_per_step": out_h_full.numel() * es,
                        "includes": "pinned-host q/k/v upload, attention, output all-gather (N>1), output download, sync"},
                "gpu_launches": int(launches), "launch_shape": dict(shape), "device_status": status,
                "clocks": clocks.summary()}
        if world == 1 and not args.no_cpu_baseline:
            smp = CpuReferenceSample(full)
            probe = smp.step()
            n = max(3, min(50, int(15.0 / max(probe, 1e-3))))
            line["cpu_baseline"] = {"value": smp.run(n, 1), "unit": "steps/s", "cores": smp.cores, "kind": "port",
                                    "sample": smp.describe(n)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
