"""Times the reference's OWN CUDA kernel (attention.cu compiled unmodified for sm_100a into
oracle/_ref, launched with both of its launch settings, kernel_launch_utils.h:135-180) next to
this engine on the four fp32/fp16 configurations of the benchmark definition, at the last
decode step, and asserts that the engine is the faster of the two.

Protocol, the same for both kernels: enough replicas of the caches to exceed the 126 MB L2
several times, used round-robin, so every launch streams from HBM; warm-up; CUDA events around
a run of back-to-back launches on one stream.  The engine is timed a second time from a CUDA
graph replay of the same launches (no host work between them); the assertion uses the slower,
per-call number.  The reference cannot run the bf16 long-sequence configuration at all (no
bf16, scores of the whole sequence in 48 KB of shared memory, 32-bit offsets), so it is absent.
"""
from dataclasses import replace

import pytest
import torch

from fastforwardattention_b200.workloads import CONFIGS, device_prompt_kv, device_step_qkv
from tests import ref_kernel
from tests.helpers import report
from tests.ref_kernel import _p

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernel.available(), reason="oracle/_ref/libffa_ref.so not built")]

NAMES = ["opt13b-fp32-b1", "opt13b-fp16-b10", "gptj-fp16-b8", "prune-fp16-b10-p1e-3"]


def _timed(run, n):
    run(n)                                   # warm-up: every replica once more
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    run(n)
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / n * 1e3       # us per launch


def measure(name):
    from fastforwardattention_b200 import FastForwardAttn

    dev = torch.device("cuda:0")
    w = CONFIGS[name]
    t = w.max_len - 1
    alg = w.dtype.itemsize * w.B * w.H * w.Dh * (2 * t + 6)
    nrep = max(2, min(12, -(-int(500e6) // alg)))
    steps = 4 * nrep
    q, k, v = device_step_qkv(w, 1, dev)[0]               # the pruning configuration keeps its queries aligned with the peaked keys
    out = torch.zeros(w.B, w.H, w.Dh, dtype=w.dtype, device=dev)
    row = {"workload": name, "MB": alg / 1e6}
    for launch in ("optimized", "ft_default"):
        refs = []
        for r in range(nrep):
            K, V = device_prompt_kv(w if w.peaked else replace(w, seed=w.seed + r), dev)   # peaked keys stay aligned with the queries
            rk = ref_kernel.ReferenceKernel(K, V, w.max_len, launch)
            rk.k_cache[..., w.prompt:, :].normal_()       # rows the decode steps would have written
            rk.v_cache[:, :, w.prompt:].normal_()
            refs.append(rk)
            del K, V

        def run_ref(n):
            for i in range(n):
                rk = refs[i % nrep]
                # the reference launches on the legacy default stream, which is torch's current stream here
                rc = rk.L.ffa_ref_attention(rk.es, rk.B, rk.H, rk.Dh, rk.Lmax, float(w.scale), int(t), _p(q), _p(k), _p(v),
                                            _p(rk.k_cache), _p(rk.v_cache), _p(out), None, float(w.p), rk.tpv, rk.tpk, rk.tpb, 1)
                assert rc == 0

        row[launch] = _timed(run_ref, steps)
        del refs
        torch.cuda.empty_cache()
    engs = []
    for r in range(nrep):
        K, V = device_prompt_kv(w if w.peaked else replace(w, seed=w.seed + r), dev)   # peaked keys stay aligned with the queries
        engs.append(FastForwardAttn(K, V, w.max_len, False))
        kc, vc = engs[-1].get_cache()
        kc[:, :, w.prompt:].normal_()
        vc[:, :, w.prompt:].normal_()
        del K, V

    def run_eng(n):
        for i in range(n):
            engs[i % nrep].attention(q, k, v, w.scale, t, w.p, out=out)

    row["engine"] = _timed(run_eng, steps)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run_eng(1)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run_eng(steps)
    row["engine_graph"] = _timed(lambda n: g.replay(), 1) / steps
    assert all(e.device_status() == 0 for e in engs)
    return row


def test_engine_is_faster_than_the_reference_kernel_on_its_own_configurations():
    rows = [measure(n) for n in NAMES]
    lines = ["", "reference kernel (attention.cu, sm_100a) vs this engine, us per decode step at the last step:",
             f"{'workload':24s} {'MB':>7s} {'ref optimized':>14s} {'ref FT default':>15s} {'engine':>9s} {'engine, graph':>14s} {'speed-up':>9s}"]
    for r in rows:
        best = min(r["optimized"], r["ft_default"])
        lines.append(f"{r['workload']:24s} {r['MB']:7.1f} {r['optimized']:14.1f} {r['ft_default']:15.1f} {r['engine']:9.1f} "
                     f"{r['engine_graph']:14.1f} {best / r['engine_graph']:8.1f}x")
    for line in lines[1:]:
        report(line)
    for r in rows:
        assert r["engine"] < min(r["optimized"], r["ft_default"]), r
