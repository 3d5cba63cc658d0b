"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Gates (max abs error against the reference's torch function on identical seeded inputs):
fp32 <= 1e-6, fp16 / bf16 <= 2e-3.  For 16-bit types the same-dtype torch function is itself
a noisy statement of the result (it rounds scores, scaled scores and probabilities to the
storage type); each comparison therefore also measures that oracle's own distance to an fp64
evaluation and, in exact mode, checks the engine against the fp32 up-cast of the contract,
where the gate is one unit in the last place.  The torch-rounding mode is held to the 2e-3
gate against the same-dtype function directly.
"""
import math

import pytest
import torch

from fastforwardattention_b200 import capi
from fastforwardattention_b200.workloads import CONFIGS, Workload, device_prompt_kv, prompt_kv, step_qkv
from oracle import ffa_oracle as O
from tests.cabi_engine import CAbiEngine
from tests.helpers import TOL, ULP, assert_close_ulp, golden_names, load_golden, max_err, report, same_dtype_gate

pytestmark = pytest.mark.gpu

# ------------------------------------------------------------------------------------------
# golden fixtures (outputs of the reference's own function text)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("use_default", [False, True])
@pytest.mark.parametrize("name", golden_names())
def test_golden_vectors(name, use_default):
    g = load_golden(name)
    dt = g["dtype"]
    Lp, n = g["prompt"], len(g["steps"])
    eng = CAbiEngine(g["K"], g["V"], Lp + n, use_default=use_default)
    orc64 = O.DecodeOracle(g["K"], g["V"], Lp + n, compute_dtype=torch.float64)
    for i, (q, k, v, want) in enumerate(g["steps"]):
        t = Lp + i
        got = eng.attention(q, k, v, g["scale"], t)
        ref64 = orc64.step(q, k, v, g["scale"], t)
        assert_close_ulp(got, ref64, dt, f"{name} step {i} vs fp64")
        if dt == torch.float32:
            assert max_err(got, want) <= TOL[dt], (name, i, max_err(got, want))
        else:
            same_dtype_gate(got, want, ref64, dt, f"{name} step {i}")
    assert eng.status() == 0
    # appended rows hold k/v bit-exactly, rows past the last step were never touched
    for i, (q, k, v, _) in enumerate(g["steps"]):
        assert torch.equal(eng.k_cache[:, :, Lp + i].cpu(), k[:, :, 0])
        assert torch.equal(eng.v_cache[:, :, Lp + i].cpu(), v[:, :, 0])
    assert torch.equal(eng.k_cache[:, :, :Lp].cpu(), g["K"])


@pytest.mark.parametrize("name", [n for n in golden_names() if not n.startswith("f32")])
def test_golden_vectors_torch_rounding_mode(name):
    g = load_golden(name)
    dt = g["dtype"]
    Lp, n = g["prompt"], len(g["steps"])
    eng = CAbiEngine(g["K"], g["V"], Lp + n)
    eng.set_mode(capi.MODE_ROUND_LIKE_TORCH)
    for i, (q, k, v, want) in enumerate(g["steps"]):
        got = eng.attention(q, k, v, g["scale"], Lp + i)
        err = (got.double().cpu() - want.double()).abs()
        # 2e-3, or one unit in the last place where the value itself is large
        bound = torch.clamp(ULP[dt] * want.double().abs(), min=TOL[dt])
        assert (err <= bound).all(), (name, i, err.max().item())
    assert eng.status() == 0


# ------------------------------------------------------------------------------------------
# the benchmark configurations, driven step by step like example.py:30-46
# ------------------------------------------------------------------------------------------
def run_config(w: Workload, step_filter, mode=capi.MODE_EXACT, use_default=False, prune_path=0):
    K, V = prompt_kv(w)
    eng = CAbiEngine(K, V, w.max_len, use_default=use_default)
    eng.set_mode(mode)
    eng.set_prune_path(prune_path)
    orc = O.DecodeOracle(K, V, w.max_len)
    N = w.B * w.H
    worst = {"same": 0.0, "noise": 0.0, "f64": 0.0}
    for t, q, k, v in step_qkv(w):
        got = eng.attention(q, k, v, w.scale, t)
        if not step_filter(t - w.prompt):
            orc.append(k, v, t)
            continue
        same = orc.step(q, k, v, w.scale, t)
        ref64 = O.attention_reference(q.view(N, 1, w.Dh), orc.K[:, : t + 1], orc.V[:, : t + 1], w.scale,
                                      torch.float64).view(w.B, w.H, w.Dh)
        if mode == capi.MODE_EXACT:
            assert_close_ulp(got, ref64, w.dtype, f"{w.name} t={t} vs fp64")
            if w.dtype == torch.float32:
                e = max_err(got, same)
                assert e <= TOL[w.dtype], (w.name, t, e)
                noise = max_err(same, ref64)
            else:
                e, noise = same_dtype_gate(got, same, ref64, w.dtype, f"{w.name} t={t}")
        else:
            e, noise = max_err(got, same), max_err(same, ref64)
            assert e <= TOL[w.dtype], (w.name, t, e, noise)
        worst["same"], worst["noise"] = max(worst["same"], e), max(worst["noise"], noise)
        worst["f64"] = max(worst["f64"], max_err(got, ref64))
    assert eng.status() == 0
    last = w.max_len - 1
    assert torch.equal(eng.k_cache.view(N, w.max_len, w.Dh)[:, : last + 1].cpu(), orc.K[:, : last + 1])
    assert torch.equal(eng.v_cache.view(N, w.max_len, w.Dh)[:, : last + 1].cpu(), orc.V[:, : last + 1])
    report(f"[parity] {w.name} mode={'exact' if mode == capi.MODE_EXACT else 'round_like_torch'} path={prune_path}: "
           f"max|engine - same-dtype torch| = {worst['same']:.3e} (gate {TOL[w.dtype]:.0e}), same-dtype torch vs fp64 = "
           f"{worst['noise']:.3e}, max|engine - fp64| = {worst['f64']:.3e}")
    return worst


def test_config_opt13b_fp32_all_steps():
    run_config(CONFIGS["opt13b-fp32-b1"], lambda i: True)


def test_config_opt13b_fp16():
    run_config(CONFIGS["opt13b-fp16-b10"], lambda i: i < 4 or i % 32 == 0 or i >= 252)


def test_config_gptj_fp16():
    run_config(CONFIGS["gptj-fp16-b8"], lambda i: i < 3 or i % 32 == 0 or i >= 126)


@pytest.mark.parametrize("x", [512, 2048])
def test_config_long_bf16(x):
    w = CONFIGS[f"long-{x}"]
    run_config(w, lambda i: i in (0, 1, 64, 127))


@pytest.mark.parametrize("path", [1, 2], ids=["cluster-kernel", "streaming-kernel"])
@pytest.mark.parametrize("x", [512, 2048])
def test_config_long_bf16_torch_rounding_mode(x, path):
    w = CONFIGS[f"long-{x}"]
    run_config(w, lambda i: i in (0, 127), mode=capi.MODE_ROUND_LIKE_TORCH, prune_path=path)


def test_config_fp16_torch_rounding_mode():
    run_config(CONFIGS["opt13b-fp16-b10"], lambda i: i in (0, 255), mode=capi.MODE_ROUND_LIKE_TORCH)


def test_default_launch_rule_matches():
    run_config(CONFIGS["opt13b-fp16-b10"], lambda i: i in (0, 100), use_default=True)


# ------------------------------------------------------------------------------------------
# full-size long sequence: sampled (batch, head) pairs against the oracle + properties
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("x", [8192, 32768])
def test_long_sequence_full_size_sampled_heads(x):
    w = CONFIGS[f"long-{x}"]
    dev = torch.device("cuda:0")
    K, V = device_prompt_kv(w, dev)
    eng = CAbiEngine(K, V, w.max_len)
    N = w.B * w.H
    g = torch.Generator().manual_seed(x)
    pick = torch.randperm(N, generator=g)[:6]
    Ks = K.view(N, w.prompt, w.Dh)[pick.to(dev)].cpu()
    Vs = V.view(N, w.prompt, w.Dh)[pick.to(dev)].cpu()
    del K, V
    orc = O.DecodeOracle(Ks[:, None], Vs[:, None], w.max_len)
    outs = {}
    worst = {"same": 0.0, "noise": 0.0, "f64": 0.0}
    for shape in ({}, {"tile_rows": 32, "stages": 2, "ctas_per_sm": 3}):
        eng.set_launch(**shape)
        for i, t in enumerate((w.prompt, w.prompt + 1, w.max_len - 1)):
            gq = torch.Generator().manual_seed(1000 * x + t)
            q = torch.randn(N, w.Dh, generator=gq).to(w.dtype)
            k = torch.randn(N, w.Dh, generator=gq).to(w.dtype)
            v = torch.randn(N, w.Dh, generator=gq).to(w.dtype)
            if t == w.max_len - 1:
                # rows between the second step and the last were never appended: fill them
                fill = torch.randn(N, w.max_len - 1 - (w.prompt + 2), w.Dh, generator=torch.Generator().manual_seed(7)).to(w.dtype)
                eng.k_cache.view(N, w.max_len, w.Dh)[:, w.prompt + 2: w.max_len - 1] = fill.to(dev)
                eng.v_cache.view(N, w.max_len, w.Dh)[:, w.prompt + 2: w.max_len - 1] = (0.5 * fill).to(dev)
                orc.K[:, w.prompt + 2: w.max_len - 1] = fill[pick]
                orc.V[:, w.prompt + 2: w.max_len - 1] = (0.5 * fill)[pick]
            got = eng.attention(q, k, v, w.scale, t)
            same = orc.step(q[pick], k[pick], v[pick], w.scale, t)[:, 0]
            ref64 = O.attention_reference(q[pick][:, None], orc.K[:, : t + 1], orc.V[:, : t + 1], w.scale, torch.float64)
            gs = got.view(N, w.Dh)[pick.to(dev)]
            assert_close_ulp(gs, ref64, w.dtype, f"{w.name} t={t} sampled heads vs fp64")
            err, noise = same_dtype_gate(gs, same, ref64, w.dtype, f"{w.name} t={t}")
            # at the benchmarked lengths the stated gate holds as it stands, without the allowance for the oracle's own noise
            assert err <= TOL[w.dtype], (w.name, t, err, noise)
            worst["same"], worst["noise"] = max(worst["same"], err), max(worst["noise"], noise)
            worst["f64"] = max(worst["f64"], max_err(gs, ref64))
            outs.setdefault(i, []).append(got.float().cpu())
    report(f"[parity] {w.name} mode=exact, 6 sampled pairs x 3 steps x 2 launch shapes: max|engine - same-dtype torch| = "
           f"{worst['same']:.3e} (gate {TOL[w.dtype]:.0e}, un-widened), same-dtype torch vs fp64 = {worst['noise']:.3e}, "
           f"max|engine - fp64| = {worst['f64']:.3e}")
    # the result must not depend on how the work was cut (different tiles, ring, grid)
    for i, (a, b) in outs.items():
        assert (a - b).abs().max().item() <= 2 * ULP[w.dtype] * max(1.0, a.abs().max().item())
    # property: constant V rows give that constant back whatever the scores (softmax sums to 1)
    eng.set_launch()
    eng.v_cache.view(N, w.max_len, w.Dh)[:] = 0.375
    q = torch.randn(N, w.Dh, generator=g).to(w.dtype)
    k = torch.randn(N, w.Dh, generator=g).to(w.dtype)
    v = torch.full((N, w.Dh), 0.375, dtype=w.dtype)
    got = eng.attention(q, k, v, w.scale, w.max_len - 1)
    assert (got.float() - 0.375).abs().max().item() <= 2.0 ** -9
    assert eng.status() == 0


# ------------------------------------------------------------------------------------------
# edge cases: tile edges, forced launch shapes, masks, per-sample lengths
# ------------------------------------------------------------------------------------------
def small_case(dt, B, H, Dh, Lp, Lmax, seed):
    g = torch.Generator().manual_seed(seed)
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    return g, K, V


def qkv(g, B, H, Dh, dt):
    return tuple(torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))


@pytest.mark.parametrize("dt,Dh", [(torch.float32, 64), (torch.float16, 64), (torch.bfloat16, 128), (torch.float16, 80),
                                   (torch.float32, 256), (torch.float16, 256), (torch.float32, 80), (torch.bfloat16, 80)])
@pytest.mark.parametrize("shape", [dict(tile_rows=8, stages=2, consumer_warps=1, grid=1),
                                   dict(tile_rows=16, stages=3, consumer_warps=4),
                                   dict(tile_rows=64, stages=2, consumer_warps=8, ctas_per_sm=1),
                                   dict(tile_rows=8, stages=5, consumer_warps=7, ctas_per_sm=4)])
def test_tile_edges_and_forced_shapes(dt, Dh, shape):
    B, H = 2, 3
    R = shape["tile_rows"]
    for Lp in (0, 1, R - 1, R, R + 1, 3 * R - 1, 3 * R, 5 * R + 3):
        steps = 2
        g, K, V = small_case(dt, B, H, Dh, Lp, Lp + steps, 100 + Lp)
        eng = CAbiEngine(K, V, Lp + steps)
        eng.set_launch(**shape)
        orc = O.DecodeOracle(K, V, Lp + steps, compute_dtype=torch.float64)
        for i in range(steps):
            q, k, v = qkv(g, B, H, Dh, dt)
            got = eng.attention(q, k, v, 1 / math.sqrt(Dh), Lp + i)
            ref = orc.step(q, k, v, 1 / math.sqrt(Dh), Lp + i)
            assert_close_ulp(got, ref, dt, f"{dt} Dh={Dh} {shape} Lp={Lp} step {i}")
        assert eng.status() == 0


def test_canary_rows_are_untouched():
    dt, B, H, Dh, Lp, Lmax = torch.float16, 2, 4, 64, 50, 90
    g, K, V = small_case(dt, B, H, Dh, Lp, Lmax, 3)
    eng = CAbiEngine(K, V, Lmax)
    for i in range(5):
        q, k, v = qkv(g, B, H, Dh, dt)
        eng.attention(q, k, v, 0.125, Lp + i)
    assert (eng.k_cache[:, :, Lp + 5:] == 777.0).all() and (eng.v_cache[:, :, Lp + 5:] == 777.0).all()
    # last legal row
    q, k, v = qkv(g, B, H, Dh, dt)
    eng.attention(q, k, v, 0.125, Lmax - 1)
    assert torch.equal(eng.k_cache[:, :, Lmax - 1].cpu(), k[:, :, 0])
    assert (eng.k_cache[:, :, Lp + 5: Lmax - 1] == 777.0).all()
    with pytest.raises(capi.FfaError) as e:
        eng.attention(q, k, v, 0.125, Lmax)
    assert e.value.code == -3
    with pytest.raises(capi.FfaError):
        eng.attention(q, k, v, 0.125, Lp, p=1.5)
    assert eng.status() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("p", [0.0, 1e-3])
@pytest.mark.parametrize("path", [1, 2], ids=["cluster-kernel", "streaming-kernel"])
def test_left_padding_mask(dt, p, path):
    """The 9-argument overload of the reference: keys below seq_lengths[b] are masked
    (attention.cu:814-817, 1054, 1112-1113)."""
    B, H, Dh, Lp, Lmax = 4, 3, 64, 70, 75
    g, K, V = small_case(dt, B, H, Dh, Lp, Lmax, 21)
    first = torch.tensor([0, 13, 69, 70], dtype=torch.int32)
    eng = CAbiEngine(K, V, Lmax)
    eng.set_prune_path(path)
    eng.set_launch(tile_rows=16)
    orc = O.DecodeOracle(K, V, Lmax)
    for i in range(3):
        t = Lp + i
        q, k, v = qkv(g, B, H, Dh, dt)
        got = eng.attention(q, k, v, 0.125, t, p=p, seq_lengths=first, right_or_no_padding=False, want_mask=p > 0)
        orc.append(k, v, t)
        fk = first.repeat_interleave(H)
        want, kept, info = O.pruned_attention(q.view(B * H, Dh), orc.K[:, : t + 1], orc.V[:, : t + 1], 0.125, p,
                                              first_key=fk, eps=1e-6 if p > 0 else 0.0)
        tol = {torch.float32: 2e-6, torch.float16: 2e-3, torch.bfloat16: 8e-3}[dt]
        assert max_err(got.view(B * H, Dh), want) <= tol
        if p > 0:
            mine = eng.kept(t)
            diff = mine != kept
            assert int(diff.sum()) <= info["borderline"], (int(diff.sum()), info)
    assert eng.status() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_per_sample_lengths_right_padding(dt):
    """do_attention<T> of c_ffa_api.h:17-20: sample b appends at row seq_lengths[b] and attends
    rows 0..seq_lengths[b] (attention.cu:808-812)."""
    B, H, Dh, Lmax = 4, 2, 128, 100
    g = torch.Generator().manual_seed(4)
    K = torch.randn(B, H, Lmax, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lmax, Dh, generator=g).to(dt)
    lens = torch.tensor([0, 17, 64, 99], dtype=torch.int32)
    eng = CAbiEngine(K, V, Lmax)
    eng.set_launch(tile_rows=16)
    q, k, v = qkv(g, B, H, Dh, dt)
    got = eng.attention(q, k, v, Dh ** -0.5, Lmax - 1, seq_lengths=lens, right_or_no_padding=True)
    for b in range(B):
        L = int(lens[b])
        Kb = torch.cat([K[b, :, :L], k[b]], dim=1)
        Vb = torch.cat([V[b, :, :L], v[b]], dim=1)
        ref = O.attention_reference(q[b], Kb, Vb, Dh ** -0.5, torch.float64)
        assert_close_ulp(got[b], ref, dt, f"sample {b}")
        assert torch.equal(eng.k_cache[b, :, L].cpu(), k[b, :, 0])
        assert torch.equal(eng.k_cache[b, :, L + 1:].cpu(), K[b, :, L + 1:])
    assert eng.status() == 0
    # a length outside the cache is reported, not written
    bad = torch.tensor([0, 17, 100, 5], dtype=torch.int32)
    eng.attention(q, k, v, Dh ** -0.5, Lmax - 1, seq_lengths=bad, right_or_no_padding=True)
    assert eng.status() & 2
    # a tight bound on the lengths (what a host that tracks them passes) gives the same result ...
    short = torch.tensor([0, 17, 30, 9], dtype=torch.int32)
    eng2 = CAbiEngine(K, V, Lmax)
    a = eng2.attention(q, k, v, Dh ** -0.5, 30, seq_lengths=short, right_or_no_padding=True)
    eng3 = CAbiEngine(K, V, Lmax)
    b = eng3.attention(q, k, v, Dh ** -0.5, Lmax - 1, seq_lengths=short, right_or_no_padding=True)
    for bb in range(B):
        L = int(short[bb])
        ref = O.attention_reference(q[bb], torch.cat([K[bb, :, :L], k[bb]], dim=1), torch.cat([V[bb, :, :L], v[bb]], dim=1),
                                    Dh ** -0.5, torch.float64)
        assert_close_ulp(a[bb], ref, dt, f"tight bound, sample {bb}")
        assert_close_ulp(b[bb], ref, dt, f"loose bound, sample {bb}")
    assert eng2.status() == 0 and eng3.status() == 0
    # ... and a length above the stated bound is refused and reported, never cut short
    eng2.attention(q, k, v, Dh ** -0.5, 29, seq_lengths=short, right_or_no_padding=True)
    assert eng2.status() & 2
    assert torch.equal(eng2.k_cache[2, :, 31:].cpu(), K[2, :, 31:])


# ------------------------------------------------------------------------------------------
# pruning: the kept set must equal the reference rule's
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("path", [1, 2], ids=["cluster-kernel", "streaming-kernel"])
@pytest.mark.parametrize("name", ["prune-fp16-b10-p1e-4", "prune-fp16-b10-p1e-3"])
def test_pruning_workload_kept_set(name, path):
    w = CONFIGS[name]
    K, V = prompt_kv(w)
    eng = CAbiEngine(K, V, w.max_len)
    eng.set_prune_path(path)
    orc = O.DecodeOracle(K, V, w.max_len)
    N = w.B * w.H
    checked = 0
    for t, q, k, v in step_qkv(w):
        i = t - w.prompt
        got = eng.attention(q, k, v, w.scale, t, p=w.p, want_mask=True)
        orc.append(k, v, t)
        if not (i < 2 or i % 64 == 0 or i == w.steps - 1):
            continue
        want, kept, info = O.pruned_attention(q.view(N, w.Dh), orc.K[:, : t + 1], orc.V[:, : t + 1], w.scale, w.p)
        assert info["borderline"] == 0, info          # the workload has a wide logit gap
        assert torch.equal(eng.kept(t), kept), f"{name} t={t}: kept sets differ"
        assert max_err(got.view(N, w.Dh), want) <= TOL[w.dtype]
        assert 0.03 < info["kept_fraction"] < 0.08    # the 5 % peaks survive, nothing else
        checked += 1
    assert checked >= 6 and eng.status() == 0


@pytest.mark.parametrize("path", [1, 2], ids=["cluster-kernel", "streaming-kernel"])
@pytest.mark.parametrize("dt,Dh,B,H,Lp", [(torch.float32, 80, 1, 3, 333), (torch.float16, 80, 2, 2, 1500),
                                          (torch.bfloat16, 256, 1, 2, 2100), (torch.float32, 256, 1, 1, 40),
                                          (torch.float16, 128, 40, 8, 95), (torch.bfloat16, 64, 1, 1, 9000)])
def test_pruning_all_head_dims_both_paths(dt, Dh, B, H, Lp, path):
    """Slices per (batch, head) from 1 to 8, slices shorter than a tile, rounds of more than
    1024 rows, head_dim 80: kept set and output against the restated rule on both paths."""
    g, K, V = small_case(dt, B, H, Dh, Lp, Lp + 2, 900 + Dh + Lp)
    eng = CAbiEngine(K, V, Lp + 2)
    eng.set_prune_path(path)
    orc = O.DecodeOracle(K, V, Lp + 2)
    for i, p in enumerate((1e-3, 0.05)):
        t = Lp + i
        q, k, v = qkv(g, B, H, Dh, dt)
        q = 2.0 * q
        got = eng.attention(q, k, v, Dh ** -0.5, t, p=p, want_mask=True)
        orc.append(k, v, t)
        want, kept, info = O.pruned_attention(q.view(B * H, Dh), orc.K[:, : t + 1], orc.V[:, : t + 1], Dh ** -0.5, p)
        diff = int((eng.kept(t) != kept).sum())
        assert diff <= info["borderline"], (p, diff, info)
        tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 8e-3}[dt]
        assert max_err(got.view(B * H, Dh), want) <= tol + 0.05 * diff
        assert torch.equal(eng.v_cache[:, :, t].cpu(), v[:, :, 0]) and torch.equal(eng.k_cache[:, :, t].cpu(), k[:, :, 0])
    assert eng.status() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_pruning_straddling_scores(dt):
    """Scores spread across the threshold: sets must agree except on positions the oracle
    itself marks as within one rounding step of the threshold."""
    B, H, Dh, Lp, Lmax = 2, 4, 64, 600, 610
    g, K, V = small_case(dt, B, H, Dh, Lp, Lmax, 77)
    eng = CAbiEngine(K, V, Lmax)
    orc = O.DecodeOracle(K, V, Lmax)
    total_diff = total_border = 0
    for i, p in enumerate((1e-4, 1e-3, 1e-2, 0.2)):
        t = Lp + i
        q, k, v = qkv(g, B, H, Dh, dt)
        q = 2.5 * q
        got = eng.attention(q, k, v, 0.125, t, p=p, want_mask=True)
        orc.append(k, v, t)
        want, kept, info = O.pruned_attention(q.view(B * H, Dh), orc.K[:, : t + 1], orc.V[:, : t + 1], 0.125, p)
        diff = int((eng.kept(t) != kept).sum())
        total_diff += diff
        total_border += info["borderline"]
        assert 0.0 < info["kept_fraction"] < 1.0
        assert diff <= info["borderline"], (p, diff, info)
        tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 8e-3}[dt]
        assert max_err(got.view(B * H, Dh), want) <= tol + 0.05 * diff
    print(f"\n[prune straddle] {dt}: differing={total_diff} borderline={total_border}")
    assert eng.status() == 0


def test_bounded_wait_times_out_and_reports():
    """Failure detection on the device: a wait on a barrier that nothing completes runs out
    after its limit, the kernel returns, the status word carries the time-out bit, and the
    context stays usable (the next decode step is correct)."""
    import ctypes as C
    import time

    dt, B, H, Dh, Lp = torch.float16, 1, 2, 64, 20
    g, K, V = small_case(dt, B, H, Dh, Lp, Lp + 1, 5)
    eng = CAbiEngine(K, V, Lp + 1)
    t0 = time.time()
    capi.check(eng.L.ffa_selftest_wait_timeout(eng.plan, 50, None))
    torch.cuda.synchronize()
    assert 0.04 < time.time() - t0 < 1.5
    assert eng.status() == 1          # FFA_STATUS_WAIT_TIMEOUT, and reading clears it
    assert eng.status() == 0
    q, k, v = qkv(g, B, H, Dh, dt)
    got = eng.attention(q, k, v, 0.125, Lp)
    ref = O.DecodeOracle(K, V, Lp + 1, compute_dtype=torch.float64).step(q, k, v, 0.125, Lp)
    assert_close_ulp(got, ref, dt, "step after the timed-out wait")
    assert eng.status() == 0


@pytest.mark.parametrize("p,path", [(0.0, 0), (1e-2, 1), (1e-2, 2)], ids=["exact", "prune-cluster", "prune-streaming"])
def test_results_are_bitwise_reproducible(p, path):
    """Split partials are merged in slot order and pruning survivors are listed in row order, so
    two runs on the same inputs give the same bits whatever the CTA timing."""
    dt, B, H, Dh, Lp = torch.float16, 3, 8, 128, 3000
    g, K, V = small_case(dt, B, H, Dh, Lp, Lp + 1, 31)
    q, k, v = qkv(g, B, H, Dh, dt)
    outs = []
    for rep in range(3):
        eng = CAbiEngine(K, V, Lp + 1)
        eng.set_prune_path(path)
        eng.set_launch(tile_rows=16, ctas_per_sm=4)     # many splits per (batch, head)
        outs.append(eng.attention(2 * q, k, v, Dh ** -0.5, Lp, p=p).cpu())
        assert eng.status() == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("dt,B,H,Dh,Lp", [(torch.float32, 1, 32, 64, 999), (torch.float16, 1, 16, 256, 2047),
                                          (torch.bfloat16, 4, 32, 128, 2047), (torch.float16, 2, 3, 80, 500),
                                          (torch.float32, 1, 1, 128, 4000), (torch.bfloat16, 1, 2, 64, 7),
                                          (torch.bfloat16, 2, 4, 128, 8191), (torch.float16, 1, 4, 64, 20000)])
def test_cluster_merge_equals_merge_through_global_memory(dt, B, H, Dh, Lp):
    """Few (batch, head) pairs: the CTAs that share a pair merge inside a thread-block cluster
    through distributed shared memory.  Same partials, same order of operations as the merge
    through global memory and an arrival counter, so the two give the same bits; both are
    checked against the oracle.  With very few pairs a pair is several clusters of 8 whose leaders
    then merge through global memory: one more level, so equal within rounding instead of
    bit-identical."""
    from fastforwardattention_b200 import FastForwardAttn

    g, K, V = small_case(dt, B, H, Dh, Lp, Lp + 2, 77 + Dh)
    orc = O.DecodeOracle(K, V, Lp + 2, compute_dtype=torch.float64)
    a = FastForwardAttn(K.cuda(), V.cuda(), Lp + 2, False)
    b = FastForwardAttn(K.cuda(), V.cuda(), Lp + 2, False)
    b.set_cluster_merge(False)
    parts, parts_b = a.launch_shape(Lp)["parts_per_bh"], b.launch_shape(Lp)["parts_per_bh"]
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    for i in range(2):
        q, k, v = qkv(g, B, H, Dh, dt)
        oa = a.attention(q.cuda(), k.cuda(), v.cuda(), Dh ** -0.5, Lp + i, 0.0)
        ob = b.attention(q.cuda(), k.cuda(), v.cuda(), Dh ** -0.5, Lp + i, 0.0)
        if parts <= 8 and parts == parts_b:
            assert torch.equal(oa, ob), (parts, i)
        else:   # another cut (9 parts -> 8) or one more merge level: equal within rounding
            assert (oa.float() - ob.float()).abs().max().item() <= tol
        ref = orc.step(q, k, v, Dh ** -0.5, Lp + i)
        assert (oa.cpu().double() - ref).abs().max().item() <= tol
    assert a.device_status() == 0 and b.device_status() == 0
    if B * H <= 32 and Lp >= 500:
        assert 2 <= parts <= 8 or parts % 8 == 0        # these shapes do run as clusters


@pytest.mark.parametrize("dt,B,H,Dh,L", [(torch.bfloat16, 1, 4, 128, 131072), (torch.float16, 1, 2, 64, 500000),
                                         (torch.float32, 1, 1, 256, 200000)])
def test_very_long_sequences_exact_and_pruned(dt, B, H, Dh, L):
    """Far beyond the reference's ~8 K-token limit (its scores live in 48 KB of shared memory,
    attention.cu:660-688): 128 K to 500 K tokens, few pairs, so a pair is spread over many
    clusters.  Exact step against an fp64 evaluation; pruned step (fused kernel where a slice's
    scores fit in shared memory, the streaming kernel where they do not) against the restated rule."""
    from fastforwardattention_b200 import FastForwardAttn

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(L + Dh)
    K = torch.randn(B, H, L - 2, Dh, generator=g, device=dev).to(dt)
    V = torch.randn(B, H, L - 2, Dh, generator=g, device=dev).to(dt)
    ffa = FastForwardAttn(K, V, L, False)
    ffa.record_kept_mask(True)
    Kc, Vc = K.cpu(), V.cpu()
    del K, V
    gc = torch.Generator().manual_seed(3)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    for i, p in enumerate((0.0, 1e-2)):
        t = L - 2 + i
        q, k, v = (torch.randn(B, H, 1, Dh, generator=gc).to(dt) for _ in range(3))
        q = 3.0 * q
        got = ffa.attention(q.cuda(), k.cuda(), v.cuda(), Dh ** -0.5, t, p).cpu()
        Kc, Vc = torch.cat([Kc, k], dim=2), torch.cat([Vc, v], dim=2)
        if p == 0.0:
            ref = O.attention_reference(q.view(B * H, 1, Dh), Kc.view(B * H, t + 1, Dh), Vc.view(B * H, t + 1, Dh), Dh ** -0.5,
                                        torch.float64, chunk=1)
            assert (got.view(B * H, Dh).double() - ref).abs().max().item() <= tol
        else:
            want, kept, info = O.pruned_attention(q.view(B * H, Dh), Kc.view(B * H, t + 1, Dh), Vc.view(B * H, t + 1, Dh), Dh ** -0.5, p)
            m = ffa.get_kept_mask().cpu().view(B * H, -1).to(torch.int64) & 0xFFFFFFFF
            mine = ((m[:, :, None] >> torch.arange(32)[None, None, :]) & 1).reshape(B * H, -1)[:, : t + 1].bool()
            diff = int((mine != kept).sum())
            assert diff <= info["borderline"], (diff, info)
            assert 0 < int(kept.sum()) < kept.numel()
            assert (got.view(B * H, Dh).double() - want.double()).abs().max().item() <= tol + 0.05 * diff
    assert ffa.device_status() == 0
