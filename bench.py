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

from fastforwardattention_b200.workloads import CONFIGS, device_prompt_kv, device_step_qkv  # noqa: E402

METRIC = "decode_attention_steps_per_sec"
DTYPE_NAME = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}   # storage type; sums are fp32
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch divided by the launch's algorithmic
# bytes, from one ncu capture per kernel (the exact kernel on the bf16 head_dim-128 2048-token
# case, the cluster pruning kernel on the fp16 head_dim-64 pruning configuration, the streaming
# pruning kernel on the bf16 head_dim-128 8192-token pruning workload), scaled by the bytes a
# launch streams, which is what the kernels' traffic is proportional to.
TRAFFIC_RATIO = {"ffa_stream_kernel (one-pass)": 1.004, "ffa_prune_cluster_kernel": 0.99, "ffa_prune_stream_kernel": 1.006}
# workloads reported in the `configs` key next to the headline (kernel time only, N = 1)
EXTRA_CONFIGS = ("opt13b-fp32-b1", "opt13b-fp16-b10", "gptj-fp16-b8", "prune-fp16-b10-p1e-3", "long-512", "long-2048",
                 "long-8192", "prune-long-8192")
ROUND_LIKE_TORCH_CONFIGS = ("long-512", "long-2048")


def algorithmic_bytes(es, B, H, Dh, t, kept_frac=None):
    """K and V rows 0..t-1 read once, q/k/v read, rows t written, out written.  With pruning
    only the surviving share of the V rows is read."""
    if kept_frac is None:
        return es * B * H * Dh * (2 * t + 6)
    return es * B * H * Dh * (t + 6) + int(es * B * H * Dh * t * kept_frac)


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
    """nvidia-smi clocks and throttle reasons (read-only query), sampled every 50 ms from before
    the timed region until after it; only samples whose timestamp falls inside the window given
    to summary() are reported."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.rows = index, None, []   # an nvidia-smi id: index or GPU-<uuid>

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            time.sleep(0.4)   # let it start producing before the timed region begins
        except Exception:
            self.proc = None
        return self

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.06)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        import datetime

        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 8:
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                except ValueError:
                    continue
                self.rows.append((ts, f[1:]))

    def summary(self, t0, t1):
        rows = [r for ts, r in self.rows if t0 <= ts <= t1]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(rows[0][1]),
                "power_w_max": max(float(r[2]) for r in rows), "reasons": reasons, "samples": len(rows),
                "window": "timed steps, continued untimed with the same steps up to 0.5 s when shorter"}


class CpuReferenceSample:
    """The reference's torch function (example.py:6-7) on the host cores over a bounded sample
    of the workload: `pairs` (batch, head) pairs of the full configuration at its final
    length.  One call of step() is one evaluation over the sample; the full-workload step
    time is extrapolated by the pair count ((batch, head) pairs are independent)."""

    def __init__(self, w, pairs=128):
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
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
            "config": workload_config(w, args.gpus),
            "cpu_baseline": {"value": value, "unit": "steps/s", "cores": smp.cores, "kind": "port",
                             "sample": smp.describe(steps)},
            "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def replicas_for(w):
    """Engines a workload needs so that consecutive steps stream from HBM, not from the 126 MB L2:
    one when its KV is >= 600 MB, else enough replicas (own caches each) to reach 600 MB together."""
    kv_bytes = 2 * w.B * w.H * w.max_len * w.Dh * w.dtype.itemsize
    return 1 if kv_bytes >= 600e6 else min(16, -(-int(600e6) // kv_bytes))


def kept_fraction(engine, step):
    """Share of cached V rows that survive the threshold, counted from the kept mask of one step."""
    engine.record_kept_mask(True)
    t = step()
    m = engine.get_kept_mask().view(-1)
    bits = sum(int(((m >> i) & 1).sum()) for i in range(32))
    engine.record_kept_mask(False)
    return bits / (m.numel() // ((engine.max_len + 31) // 32) * (t + 1))


def graph_replay_ms(step, steps):
    """Records `steps` consecutive calls of step(i) in one CUDA graph and returns the device time
    of one replay divided by `steps`: no host work between the launches."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(0)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):   # other threads (NCCL watchdog) keep running
        for i in range(steps):
            step(i)
    graph.replay()
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    graph.replay()
    g1.record()
    torch.cuda.synchronize()
    return g0.elapsed_time(g1) / steps


def measure_config(name, dev, peak, mode=None, steps=32):
    """Kernel time of one workload at its last decode step: `steps` launches over rotating
    replicas replayed from a CUDA graph, CUDA events around the replay."""
    from dataclasses import replace

    from fastforwardattention_b200 import FastForwardAttn

    w = CONFIGS[name]
    nrep = replicas_for(w)
    engines = []
    for r in range(nrep):
        K, V = device_prompt_kv(w if w.peaked else replace(w, seed=w.seed + 17 * r), dev)
        engines.append(FastForwardAttn(K, V, w.max_len, False))
        kc, vc = engines[-1].get_cache()     # rows the decode steps would have filled
        kc[:, :, w.prompt:].normal_()
        vc[:, :, w.prompt:].normal_()
        if mode:
            engines[-1].set_mode(mode)
        del K, V
    qkv = device_step_qkv(w, 4, dev)
    out = torch.empty(w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
    t = w.max_len - 1

    def step(i):
        engines[i % nrep].attention(qkv[i % 4, 0], qkv[i % 4, 1], qkv[i % 4, 2], w.scale, t, w.p, out=out)
        return t

    for i in range(nrep):
        step(i)
    ms = graph_replay_ms(step, steps)
    kept = kept_fraction(engines[0], lambda: step(0)) if w.p > 0 else None
    alg = algorithmic_bytes(w.dtype.itemsize, w.B, w.H, w.Dh, t, kept)
    gbs = alg / (ms * 1e-3) / 1e9
    res = {"workload": name, "dtype": DTYPE_NAME[w.dtype], "batch": w.B, "heads": w.H, "head_dim": w.Dh, "rows": t + 1,
           "p": w.p, "mode": mode or "exact", "kernel_us": round(ms * 1e3, 2), "bytes_per_launch": alg,
           "achieved_gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "kept_v_rows": kept, "replicas": nrep,
           "launch_shape": dict(engines[0].launch_shape(t)), "device_status": max(e.device_status() for e in engines)}
    del engines
    torch.cuda.empty_cache()
    return res


def result_check(w, world, rank, engine, sharded, host_step, qkv_host, t, dev, same_dtype=False):
    """One step outside the timed regions, checked three ways: (N > 1) the gathered [B, H, Dh]
    holds this rank's own shard bit for bit and equals an NCCL all-gather of the same shards;
    the tensor the end-to-end step leaves in pinned host memory agrees with the per-call path;
    four sampled (batch, head) pairs of this rank's shard agree with the checker's float64
    evaluation of softmax(q K^T scale) V over the cache rows 0..t (torch-rounding mode: with the
    same function evaluated in the tensors' own dtype, which is what that mode reproduces)."""
    import torch.distributed as dist

    from oracle.ffa_oracle import attention_reference, pruned_attention, torch_attn_func   # the checker, not the product

    q, k, v = (qkv_host[i].to(dev) for i in range(3))
    local = engine.attention(q, k, v, w.scale, t, w.p)
    full, res = local, {"ok": True}
    if world > 1:
        full = sharded.gather(local)
        ref = torch.empty(world, w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
        dist.all_gather_into_tensor(ref.view(-1), local.contiguous().view(-1))
        ref = ref.permute(1, 0, 2, 3).reshape(w.B, world * w.H, w.Dh)
        res["own_shard_bitwise"] = bool(torch.equal(full[:, rank * w.H:(rank + 1) * w.H], local))
        res["equals_nccl_all_gather"] = bool(torch.equal(full, ref))
        res["ok"] = res["own_shard_bitwise"] and res["equals_nccl_all_gather"]
    if host_step is not None:
        # the same step again through the graphed end-to-end path (row t is rewritten with the same k, v)
        host_step.reset_row(t)
        out_host = host_step(qkv_host)
        torch.cuda.current_stream().synchronize()
        res["graphed_vs_per_call_max_diff"] = (out_host.float() - full.cpu().float()).abs().max().item()
        res["ok"] = res["ok"] and res["graphed_vs_per_call_max_diff"] <= 2e-3
        delivered = out_host.clone()
    else:
        delivered = full.cpu()
    kc, vc = engine.get_cache()
    g = torch.Generator().manual_seed(4242 + rank)
    worst = 0.0
    for _ in range(4):
        b, h = int(torch.randint(w.B, (1,), generator=g)), int(torch.randint(w.H, (1,), generator=g))
        Kp, Vp, qp = kc[b, h, :t + 1].cpu()[None], vc[b, h, :t + 1].cpu()[None], qkv_host[0][b, h]
        if w.p > 0:
            ref64 = pruned_attention(qp.view(1, w.Dh), Kp, Vp, w.scale, w.p)[0][0].double()   # the pruning rule, restated
        elif same_dtype:
            ref64 = torch_attn_func(qp.view(1, 1, w.Dh), Kp, Vp, w.scale)[0, 0].double()
        else:
            ref64 = attention_reference(qp.view(1, 1, w.Dh), Kp, Vp, w.scale, torch.float64)[0]
        worst = max(worst, (delivered[b, rank * w.H + h].double() - ref64).abs().max().item())
    tol = 1e-6 if w.dtype == torch.float32 else 2e-3
    res.update({"max_err": worst, "tolerance": tol, "pairs_checked_per_rank": 4,
                "against": "the restated pruning rule on the cache rows" if w.p > 0 else
                "softmax(q K^T scale) V on the cache rows, evaluated by torch in the tensors' dtype" if same_dtype else
                "float64 evaluation of softmax(q K^T scale) V on the cache rows"})
    res["ok"] = res["ok"] and worst <= tol
    return res


def workload_config(w, n):
    return {"workload": w.name, "batch": w.B, "heads": w.H, "head_dim": w.Dh, "prompt": w.prompt,
            "decode_steps": w.steps, "final_len": w.max_len, "p": w.p,
            "parallelism": f"heads sharded over {n} GPU(s), {w.H // n} heads each" if n > 1 else "single GPU",
            "l2": "inputs larger than L2: every step streams the whole KV cache shard from HBM"
                  if 2 * w.B * (w.H // n) * w.max_len * w.Dh * w.dtype.itemsize >= 600e6 else
                  "KV shard below 600 MB: steps rotate over engine replicas (>= 600 MB of caches together), "
                  "so every step streams from HBM; no flush kernel"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="long-32768", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="exact", choices=["exact", "round_like_torch"],
                    help="round_like_torch: the engine's torch-rounding mode (reproduces the rounding points of torch's same-dtype "
                         "path; checked against that function instead of the float64 evaluation); single GPU, p = 0 workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the `configs` key (the other configurations, N = 1)")
    ap.add_argument("--gather", choices=["peer", "nccl"], default="peer",
                    help="N > 1: output all-gather by the engine's peer-memory kernel (default) or by NCCL")
    args = ap.parse_args()
    full = CONFIGS[args.workload]
    if args.impl == "reference":
        return run_reference(args, full)

    if args.mode != "exact" and (args.gpus != 1 or full.p > 0):
        raise SystemExit("--mode round_like_torch: single GPU and a workload without a pruning threshold")
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
    # Engines: one for the default workload.  A workload whose KV shard is not several times the
    # 126 MB L2 gets replicas with their own caches, used round-robin, so that every timed step
    # streams from HBM without a flush kernel in between (a zero-fill flush leaves dirty lines
    # whose write-back then competes with the step being timed).
    nrep = replicas_for(w)
    from dataclasses import replace

    sharded, engines = [], []
    for r in range(nrep):
        # (the pruning workload keeps one seed: its step queries must stay aligned with the peaked keys)
        K, V = device_prompt_kv(w if w.peaked else replace(w, seed=w.seed + 17 * r), dev)
        if world > 1:
            sharded.append(ShardedFastForwardAttn(K, V, w.max_len, False))
            engines.append(sharded[-1].engine)
        else:
            engines.append(FastForwardAttn(K, V, w.max_len, False))
        if args.mode != "exact":
            engines[-1].set_mode(args.mode)
        del K, V
    torch.cuda.empty_cache()
    gather_kind = "none"
    if world > 1:
        peer_ok = args.gather == "peer" and all([s.enable_peer_gather() for s in sharded])
        gather_kind = "peer-memory kernel" if peer_ok else "nccl all_gather_into_tensor"
    shape = engines[0].launch_shape(w.max_len - 1)

    total = max(args.warmup + args.steps, nrep)   # the end-to-end legs warm every replica once
    qkv_d = device_step_qkv(w, total, dev)
    qkv_h = qkv_d.cpu().pin_memory()
    out_d = torch.empty(w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
    stage = torch.empty(3, w.B, w.H, 1, w.Dh, dtype=w.dtype, device=dev)
    out_h = torch.empty(w.B, w.H * world, w.Dh, dtype=w.dtype).pin_memory()
    t_of = lambda s: w.prompt + ((s // nrep) % w.steps)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def resident_step(s):
        engines[s % nrep].attention(qkv_d[s, 0], qkv_d[s, 1], qkv_d[s, 2], w.scale, t_of(s), w.p, out=out_d)

    def eager_e2e_step(s):
        stage.copy_(qkv_h[s], non_blocking=True)
        if world > 1:
            o = sharded[s % nrep].attention(stage[0], stage[1], stage[2], w.scale, t_of(s), w.p, gather=True)
        else:
            o = engines[s % nrep].attention(stage[0], stage[1], stage[2], w.scale, t_of(s), w.p)
        out_h.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the caller consumes the result every step

    # The end-to-end step of the public API: GraphedHostStep / ShardedFastForwardAttn.graphed_step -- one
    # upload of the step's q/k/v from pinned host memory, one replay of a CUDA graph holding the attention
    # launch (row index in device memory), the peer-memory all-gather (N > 1) and the download of the
    # result into pinned host memory, then the stream sync with which the caller takes the result.
    host_steps = None
    if world == 1 or gather_kind == "peer-memory kernel":
        from fastforwardattention_b200 import GraphedHostStep

        host_steps = [sharded[r].graphed_step(w.scale, w.prompt, w.p) if world > 1 else
                      GraphedHostStep(engines[r], w.scale, w.prompt, w.p) for r in range(nrep)]

    def e2e_step(s):
        if host_steps is None:
            return eager_e2e_step(s)
        hs = host_steps[s % nrep]
        if hs.next_row != t_of(s):
            hs.reset_row(t_of(s))
        hs(qkv_h[s])
        torch.cuda.current_stream().synchronize()   # the caller consumes hs.out_host every step
        return hs.out_host

    clocks = ClockSampler(gpu_id(dev)).start()

    # ---- leg 1: inputs resident in HBM ----
    for s in range(args.warmup):
        resident_step(s)
    barrier()
    launches0 = launch_count()
    wall0 = time.time()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        resident_step(args.warmup + i)
    stop.record()
    barrier()
    launches = launch_count() - launches0
    loop_ms = start.elapsed_time(stop)
    # keep the same load running (untimed) until the clock sampler has seen it for half a second
    while time.time() - wall0 < 0.5:
        for i in range(args.steps):
            resident_step(args.warmup + i)
        torch.cuda.synchronize()
    wall1 = time.time()
    clocks.stop()
    # the kernel's own duration for the roofline: the same K launches recorded in a CUDA graph and
    # replayed, so no host work sits between them (matters when a launch is shorter than the
    # host's per-call time); CUDA events around the replay, on the replay's stream
    graph_ms = graph_replay_ms(lambda i: resident_step(args.warmup + i), args.steps)
    # long launches: the timed region itself is the kernel time (host gaps are < 0.5 %); short ones: the replay
    use_region = loop_ms / args.steps >= 0.2
    kernel_ms = [loop_ms / args.steps if use_region else graph_ms] * args.steps
    kept_frac = None
    if w.p > 0:
        s_last = args.warmup + args.steps - 1
        kept_frac = kept_fraction(engines[s_last % nrep], lambda: (resident_step(s_last), t_of(s_last))[1])
    alg = [algorithmic_bytes(es, w.B, w.H, w.Dh, t_of(args.warmup + i), kept_frac) for i in range(args.steps)]

    # ---- leg 2: end to end with host buffers (upload, attention, gather, download, sync every step) ----
    def timed_leg(step):
        for s in range(max(min(3, args.warmup), nrep)):   # every replica's step (and its CUDA graph) has run once
            step(s)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(args.warmup + i)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    graphed_ms = timed_leg(e2e_step)
    eager_ms = timed_leg(eager_e2e_step) if host_steps is not None else graphed_ms   # same step, one API call per operation
    # Both are the public API; which is faster depends on the step: a graph saves host time per operation, but its launch
    # costs more than one kernel launch, and behind a long attention kernel the later operations' host time is hidden anyway.
    # ---- leg 3: the same step with no staging copies: the kernels read q/k/v from pinned host memory
    # and write the (gathered) result to pinned host memory in place ----
    in_place_ms = None
    if world == 1 or gather_kind == "peer-memory kernel":
        def in_place_step(s):
            q, k, v = qkv_h[s][0], qkv_h[s][1], qkv_h[s][2]
            if world > 1:
                o = engines[s % nrep].attention(q, k, v, w.scale, t_of(s), w.p)
                engines[s % nrep].peer_gather(o, out=out_h)
            else:
                engines[s % nrep].attention(q, k, v, w.scale, t_of(s), w.p, out=out_h)
            torch.cuda.current_stream().synchronize()

        in_place_ms = timed_leg(in_place_step)
    # ---- outside every timed region: is what the end-to-end step delivers the right tensor? ----
    check = result_check(w, world, rank, engines[0], sharded[0] if world > 1 else None,
                         host_steps[0] if host_steps is not None else None, qkv_h[args.warmup], w.prompt + 5, dev,
                         same_dtype=args.mode != "exact")
    status = max(e.device_status() for e in engines)

    # ---- max over ranks ----
    times = torch.tensor([loop_ms, graphed_ms, sum(kernel_ms), in_place_ms or 0.0, eager_ms, check["max_err"],
                          0.0 if check["ok"] else 1.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    loop_ms, graphed_ms, ksum_ms, in_place_ms, eager_ms, check_err, check_bad = times.tolist()
    e2e_ms, e2e_api = min((eager_ms, "per call"), (graphed_ms, "graphed"))
    check["max_err"], check["ok"] = check_err, check_bad == 0.0

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = sum(alg) / (ksum_ms * 1e-3) / 1e9          # per GPU: this rank's bytes over its kernel time
        per_launch_alg = sum(alg) / len(alg)
        kernel_name = ("ffa_prune_cluster_kernel" if args.mode != "exact" else "ffa_stream_kernel (one-pass)" if w.p == 0 else
                       "ffa_prune_stream_kernel" if w.B * w.H * w.max_len * w.Dh * es >= 1e9 else "ffa_prune_cluster_kernel")
        line = {"metric": METRIC, "value": args.steps / (loop_ms * 1e-3), "unit": "steps/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": loop_ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": DTYPE_NAME[w.dtype], "accumulate": "f32", "data": "synthetic",
                "config": dict(workload_config(full, world), **({} if args.mode == "exact" else {"mode": args.mode})),
                "hbm_gbs_all_gpus": world * sum(alg) / (loop_ms * 1e-3) / 1e9,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": achieved / 8000.0,
                             "kernel": kernel_name,
                             "kept_v_rows": kept_frac, "bytes_per_launch": per_launch_alg,
                             "avg_launch_ms": ksum_ms / args.steps,
                             "duration_from": "CUDA events around the timed steps" if use_region else
                             "CUDA events around a CUDA-graph replay of the same launches (launch shorter than host time per call)",
                             "traffic": TRAFFIC_RATIO[kernel_name] * per_launch_alg},
                "e2e": {"value": args.steps / (e2e_ms * 1e-3), "unit": "steps/s",
                        "h2d_bytes_per_step": 3 * w.B * w.H * w.Dh * es, "d2h_bytes_per_step": out_h.numel() * es,
                        "includes": "pinned-host q/k/v upload, attention, output all-gather (N>1), output download, sync",
                        "api": "the faster of the two below: " + e2e_api,
                        "gather": gather_kind + (" (pushed from the attention kernel's epilogue, then wait-and-collect)"
                                                 if gather_kind == "peer-memory kernel" and w.p == 0 else ""),
                        "per_call": {"value": args.steps / (eager_ms * 1e-3), "unit": "steps/s",
                                     "what": "upload, [Sharded]FastForwardAttn.attention(gather=True at N>1), download, sync: one host call each"},
                        "graphed": None if host_steps is None else {
                            "value": args.steps / (graphed_ms * 1e-3), "unit": "steps/s",
                            "what": "GraphedHostStep / ShardedFastForwardAttn.graphed_step: one upload + one CUDA-graph replay "
                                    "(attention, gather, download) + sync"},
                        "in_place": None if not in_place_ms else {
                            "value": args.steps / (in_place_ms * 1e-3), "unit": "steps/s",
                            "what": "same step without staging copies: kernels read q/k/v from, and write the result to, "
                                    "pinned host memory over PCIe"}},
                "gpu_launches": int(launches), "launch_shape": dict(shape), "device_status": status,
                "clocks": clocks.summary(wall0, wall1), "replicas": nrep,
                ("gather_check" if world > 1 else "result_check"): check}
        if world == 1 and not args.no_cpu_baseline:
            smp = CpuReferenceSample(full)
            probe = smp.step()
            n = max(3, min(50, int(15.0 / max(probe, 1e-3))))
            line["cpu_baseline"] = {"value": smp.run(n, 1), "unit": "steps/s", "cores": smp.cores, "kind": "port",
                                    "sample": smp.describe(n)}
        if world == 1 and not args.no_configs:
            # the other configurations of the benchmark definition, kernel time only (a few seconds together)
            del host_steps, engines, sharded
            torch.cuda.empty_cache()
            line["configs"] = [measure_config(n, dev, peak) for n in EXTRA_CONFIGS]
            line["configs"] += [measure_config(n, dev, peak, mode="round_like_torch") for n in ROUND_LIKE_TORCH_CONFIGS]
        print(json.dumps(line))
    if world > 1:
        for sh in sharded:
            sh.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
