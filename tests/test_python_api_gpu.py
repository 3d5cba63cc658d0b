"""The Python class, driven the way the reference's example.py and HF forks drive it."""
import math

import pytest
import torch

from oracle import ffa_oracle as O

pytestmark = pytest.mark.gpu


def test_example_py_loop():
    """example.py:9-46 with a seed: fp16, batch 10, 32 heads, head_dim 64, prompt 1024, 128
    steps, U[0,1) inputs, optimized launch, p = 0, max relative difference < 1e-2."""
    from ff_attention import FastForwardAttn as FFA

    torch.manual_seed(0)
    B, H, Dh, Lp, n = 10, 32, 64, 1024, 128
    dt = torch.float16
    temp = 1 / math.sqrt(Dh)
    K = torch.rand(B, H, Lp, Dh, dtype=dt).cuda()
    V = torch.rand(B, H, Lp, Dh, dtype=dt).cuda()
    ffa = FFA(K, V, Lp + n, False)
    for i in range(n):
        k = torch.rand(B, H, 1, Dh, dtype=dt).cuda()
        v = torch.rand(B, H, 1, Dh, dtype=dt).cuda()
        q = torch.rand(B, H, 1, Dh, dtype=dt).cuda()
        t = Lp + i
        out = ffa.attention(q, k, v, temp, t, 0)
        K = torch.cat([K, k], axis=-2)
        V = torch.cat([V, v], axis=-2)
        if i % 16 == 0 or i == n - 1:
            ref = O.torch_attn_func(q.view(B * H, 1, Dh).cpu(), K.view(B * H, t + 1, Dh).cpu(),
                                    V.view(B * H, t + 1, Dh).cpu(), temp)
            rel = ((ref.view(B, H, 1, Dh) - out.view(B, H, 1, Dh).cpu()).abs() / ref.view(B, H, 1, Dh)).max()
            assert rel < 1e-2
            assert (ref.view(B, H, Dh).float() - out.cpu().float()).abs().max() <= 2e-3
    assert out.shape == (B, H, Dh) and out.dtype == dt
    assert ffa.device_status() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_overloads_and_get_cache(dt):
    """modeling_opt.py:201-226 / modeling_gptj.py:259-279 call convention: q/k/v as
    [B, 1, H*Dh], caches fetched with get_cache() and passed back, left-padding lengths."""
    from fastforwardattention_b200 import FastForwardAttn

    g = torch.Generator().manual_seed(3)
    B, H, Dh, Lp, Lmax = 3, 4, 64, 40, 44
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), Lmax, True)
    kc, vc = ffa.get_cache()
    assert kc.shape == (B, H, Lmax, Dh) and vc.shape == (B, H, Lmax, Dh)
    pads = torch.tensor([0, 7, 39], dtype=torch.int32)
    orc = O.DecodeOracle(K, V, Lmax, compute_dtype=torch.float64)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    for i in range(3):
        t = Lp + i
        q, k, v = (torch.randn(B, 1, H * Dh, generator=g).to(dt) for _ in range(3))
        orc.append(k, v, t)
        if i == 0:
            out = ffa.attention(q.cuda(), k.cuda(), v.cuda(), 0.125, t)            # p defaults to 0
        elif i == 1:
            out = ffa.attention(q.cuda(), k.cuda(), v.cuda(), kc, vc, 0.125, t, 0)
        else:
            out = ffa.attention(q.cuda(), k.cuda(), v.cuda(), kc, vc, 0.125, t, pads.cuda(), 0)
        fk = pads.repeat_interleave(H) if i == 2 else None
        want, _, _ = O.pruned_attention(q.view(B * H, Dh).double(), orc.K[:, : t + 1], orc.V[:, : t + 1], 0.125, 0.0,
                                        first_key=fk, eps=0.0)
        assert (out.view(B * H, Dh).cpu().double() - want.double()).abs().max() <= tol
        assert torch.equal(kc[:, :, t].cpu().view(B, 1, H * Dh), k)
    buf = torch.empty(B, H, Dh, dtype=dt, device="cuda")
    assert ffa.attention(q.cuda(), k.cuda(), v.cuda(), 0.125, Lmax - 1, 0.0, out=buf).data_ptr() == buf.data_ptr()
    assert ffa.device_status() == 0
    shape = ffa.launch_shape(Lp)
    assert shape["grid"] >= 1 and shape["tile_rows"] % 8 == 0


def test_errors_raise():
    from fastforwardattention_b200 import FastForwardAttn

    K = torch.zeros(1, 2, 8, 64, dtype=torch.float16, device="cuda")
    ffa = FastForwardAttn(K, K.clone(), 16, False)
    q = torch.zeros(1, 2, 1, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="curr_timestep"):
        ffa.attention(q, q, q, 0.125, 16, 0)
    with pytest.raises(RuntimeError, match="dtype"):
        ffa.attention(q.float(), q, q, 0.125, 8, 0)
    with pytest.raises(RuntimeError, match="elements"):
        ffa.attention(q[:, :1], q, q, 0.125, 8, 0)
    with pytest.raises(RuntimeError, match="max_timesteps"):
        FastForwardAttn(K, K.clone(), 4, False)
    with pytest.raises(RuntimeError, match="unsupported tensor type"):
        FastForwardAttn(K.double(), K.double(), 16, False)
    with pytest.raises(RuntimeError, match="head_dim"):
        FastForwardAttn(K[..., :48].contiguous(), K[..., :48].contiguous(), 16, False)


def test_pruning_through_python_class():
    from fastforwardattention_b200 import FastForwardAttn
    from fastforwardattention_b200.workloads import CONFIGS, prompt_kv, step_qkv
    from dataclasses import replace

    w = replace(CONFIGS["prune-fp16-b10-p1e-3"], B=2, steps=4)
    K, V = prompt_kv(w)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), w.max_len, False)
    ffa.record_kept_mask(True)
    orc = O.DecodeOracle(K, V, w.max_len)
    N = w.B * w.H
    for t, q, k, v in step_qkv(w):
        out = ffa.attention(q.cuda(), k.cuda(), v.cuda(), w.scale, t, w.p)
        orc.append(k, v, t)
        want, kept, info = O.pruned_attention(q.view(N, w.Dh), orc.K[:, : t + 1], orc.V[:, : t + 1], w.scale, w.p)
        m = ffa.get_kept_mask().cpu().view(N, -1).to(torch.int64) & 0xFFFFFFFF
        bits = ((m[:, :, None] >> torch.arange(32)[None, None, :]) & 1).reshape(N, -1)[:, : t + 1].bool()
        assert torch.equal(bits, kept)
        assert (out.view(N, w.Dh).cpu().float() - want.float()).abs().max() <= 2e-3
    assert ffa.device_status() == 0


@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
def test_cuda_graph_replay_with_device_side_step(dt):
    """A decode step captured ONCE in a CUDA graph and replayed for every token: the row index
    lives in device memory (per-sample lengths, the c_ffa_api.h:17-20 mode), so the captured
    launch parameters never change.  Removes the per-step host work that dominates the small
    configurations."""
    from fastforwardattention_b200 import FastForwardAttn

    g = torch.Generator().manual_seed(11)
    B, H, Dh, Lp, n = 2, 8, 64, 150, 6
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), Lp + n, False)
    orc = O.DecodeOracle(K, V, Lp + n, compute_dtype=torch.float64)
    q_s, k_s, v_s = (torch.zeros(B, H, 1, Dh, dtype=dt, device="cuda") for _ in range(3))
    out_s = torch.zeros(B, H, Dh, dtype=dt, device="cuda")
    rows = torch.full((B,), Lp, dtype=torch.int32, device="cuda")
    # warm-up outside capture (first call binds nothing new, but keeps capture free of lazy init)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ffa.attention_per_sample(q_s, k_s, v_s, 0.125, rows, 0.0, out=out_s)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ffa.attention_per_sample(q_s, k_s, v_s, 0.125, rows, 0.0, out=out_s)
        rows.add_(1)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3}[dt]
    for i in range(n):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        q_s.copy_(q), k_s.copy_(k), v_s.copy_(v)
        graph.replay()
        ref = orc.step(q, k, v, 0.125, Lp + i)
        assert (out_s.cpu().double() - ref).abs().max().item() <= tol, i
    assert int(rows[0]) == Lp + n and ffa.device_status() == 0
    kc, _ = ffa.get_cache()
    assert torch.equal(kc[:, :, Lp + n - 1].cpu(), k[:, :, 0])


def test_graphed_step_helper():
    from fastforwardattention_b200 import FastForwardAttn, GraphedStep

    dt = torch.bfloat16
    g = torch.Generator().manual_seed(12)
    B, H, Dh, Lp, n = 2, 4, 128, 90, 5
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), Lp + n, False)
    step = GraphedStep(ffa, Dh ** -0.5, first_row=Lp)
    orc = O.DecodeOracle(K, V, Lp + n, compute_dtype=torch.float64)
    for i in range(n):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        out = step(q.cuda(), k.cuda(), v.cuda())
        ref = orc.step(q, k, v, Dh ** -0.5, Lp + i)
        assert (out.cpu().double() - ref).abs().max().item() <= 8e-3
    with pytest.raises(RuntimeError, match="full"):
        step(q.cuda(), k.cuda(), v.cuda())
    assert ffa.device_status() == 0


def test_graphed_step_in_a_mostly_empty_cache_crosses_row_buckets():
    """The graph is recorded for a bucket of rows (the engine lays its work out for the bucket's upper
    bound, not for the whole cache) and again when the generation enters the next bucket."""
    from fastforwardattention_b200 import FastForwardAttn, GraphedStep
    from fastforwardattention_b200.graphed import row_bucket

    assert [row_bucket(r, 4096) for r in (0, 127, 128, 255, 256, 4000)] == [127, 127, 255, 255, 511, 4095]
    assert row_bucket(10, 50) == 49
    dt = torch.float16
    g = torch.Generator().manual_seed(13)
    B, H, Dh, Lp, n, Lmax = 2, 4, 64, 120, 14, 4096
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), Lmax, False)
    step = GraphedStep(ffa, Dh ** -0.5, first_row=Lp)
    orc = O.DecodeOracle(K, V, Lp + n, compute_dtype=torch.float64)
    for i in range(n):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        out = step(q.cuda(), k.cuda(), v.cuda())
        ref = orc.step(q, k, v, Dh ** -0.5, Lp + i)
        assert (out.cpu().double() - ref).abs().max().item() <= 1e-3, i
    assert sorted(step.graphs) == [127, 255]
    assert ffa.device_status() == 0
    kc, _ = ffa.get_cache()
    assert torch.equal(kc[:, :, Lp + n - 1].cpu(), k[:, :, 0])


def test_graphed_host_step_upload_graph_download():
    """The host-driven step as one upload plus one graph replay: q/k/v come from pinned host memory, the
    result lands in pinned host memory; a new generation over the same caches starts with reset_row()."""
    from fastforwardattention_b200 import FastForwardAttn, GraphedHostStep

    dt = torch.float16
    g = torch.Generator().manual_seed(14)
    B, H, Dh, Lp, n = 2, 4, 64, 200, 4
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), Lp + n, False)
    step = GraphedHostStep(ffa, Dh ** -0.5, first_row=Lp)
    for generation in range(2):
        orc = O.DecodeOracle(K, V, Lp + n, compute_dtype=torch.float64)
        if generation:
            step.reset_row(Lp)
        for i in range(n):
            qkv_host = torch.randn(3, B, H, 1, Dh, generator=g).to(dt).pin_memory()
            out = step(qkv_host)
            torch.cuda.current_stream().synchronize()
            assert out.is_pinned() and out.shape == (B, H, Dh)
            ref = orc.step(qkv_host[0], qkv_host[1], qkv_host[2], Dh ** -0.5, Lp + i)
            assert (out.double() - ref).abs().max().item() <= 1e-3, (generation, i)
    with pytest.raises(RuntimeError, match="full"):
        step(qkv_host)
    assert ffa.device_status() == 0


def test_graphed_layers_whole_token_in_one_graph():
    """A toy decoder (three layers, fp32 projections between the attention calls) replayed from
    one CUDA graph gives what the same layers give when called one by one."""
    from fastforwardattention_b200 import FastForwardAttn, GraphedLayers

    dt, B, H, Dh, Lp, n, NL = torch.float32, 2, 4, 64, 70, 4, 3
    E = H * Dh
    g = torch.Generator().manual_seed(31)
    Ks = [torch.randn(B, H, Lp, Dh, generator=g) for _ in range(NL)]
    Vs = [torch.randn(B, H, Lp, Dh, generator=g) for _ in range(NL)]
    W = [[(torch.randn(E, E, generator=g) / E ** 0.5).cuda() for _ in range(4)] for _ in range(NL)]

    def make_body(calls):
        def body(x, attend):
            for i in range(NL):
                q, k, v = ((x @ W[i][j]).view(B, H, 1, Dh) for j in range(3))
                calls.append(i)
                x = x + attend(i, q, k, v).reshape(B, E) @ W[i][3]
            return x
        return body

    graphed = [FastForwardAttn(Ks[i].cuda(), Vs[i].cuda(), Lp + n, False) for i in range(NL)]
    eager = [FastForwardAttn(Ks[i].cuda(), Vs[i].cuda(), Lp + n, False) for i in range(NL)]
    calls = []
    step = GraphedLayers(graphed, Dh ** -0.5, first_row=Lp, body=make_body(calls), example_input=torch.zeros(B, E))
    assert calls == [0, 1, 2] * 2                       # traced twice (warm-up + capture), never again
    orcs = [O.DecodeOracle(Ks[i], Vs[i], Lp + n, compute_dtype=torch.float64) for i in range(NL)]
    for t in range(n):
        x = torch.randn(B, E, generator=g)
        y = step(x.cuda()).clone()
        rows = torch.full((B,), Lp + t, dtype=torch.int32, device="cuda")
        want = make_body([])(x.cuda(), lambda i, q, k, v: eager[i].attention_per_sample(q, k, v, Dh ** -0.5, rows, 0))
        assert torch.equal(y, want)                     # same kernels, same launch shapes
        # and against the oracle, layer by layer, in float64
        xr = x.double()
        for i in range(NL):
            Wd = [w.cpu().double() for w in W[i]]
            q, k, v = ((xr @ Wd[j]).view(B, H, 1, Dh) for j in range(3))
            a = orcs[i].step(q.float(), k.float(), v.float(), Dh ** -0.5, Lp + t)
            xr = xr + a.reshape(B, E).double() @ Wd[3]
        assert (y.cpu().double() - xr).abs().max().item() <= 2e-3 * xr.abs().max().item()
    assert len(calls) == 2 * NL
    with pytest.raises(RuntimeError, match="full"):
        step(x.cuda())
    assert all(e.device_status() == 0 for e in graphed)


@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
def test_adopt_prefilled_caches_and_grow(dt):
    """Prefill writes K and V straight into the cache slabs (no copy at construction); the cache
    then grows past its first length while decoding."""
    from fastforwardattention_b200 import FastForwardAttn

    g = torch.Generator().manual_seed(21)
    B, H, Dh, Lp, L0 = 2, 3, 64, 50, 53
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    kc = torch.full((B, H, L0, Dh), 7.0, dtype=dt, device="cuda")
    vc = torch.full((B, H, L0, Dh), 7.0, dtype=dt, device="cuda")
    kc[:, :, :Lp] = K.cuda()          # "prefill" writing in place
    vc[:, :, :Lp] = V.cuda()
    ffa = FastForwardAttn.adopt(kc, vc, False)
    a, b = ffa.get_cache()
    assert a.data_ptr() == kc.data_ptr() and b.data_ptr() == vc.data_ptr() and ffa.max_len == L0
    n = 9
    orc = O.DecodeOracle(K, V, Lp + n, compute_dtype=torch.float64)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3}[dt]
    for i in range(n):
        t = Lp + i
        if t >= ffa.max_len:
            with pytest.raises(RuntimeError, match="curr_timestep"):
                ffa.attention(torch.zeros(B, H, 1, Dh, dtype=dt, device="cuda"), kc[:, :, :1], kc[:, :, :1], 0.125, t, 0)
            ffa.grow(2 * ffa.max_len)
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        out = ffa.attention(q.cuda(), k.cuda(), v.cuda(), 0.125, t, 0)
        ref = orc.step(q, k, v, 0.125, t)
        assert (out.cpu().double() - ref).abs().max().item() <= tol, i
    assert ffa.max_len == 2 * L0
    nk, nv = ffa.get_cache()
    assert nk.shape == (B, H, 2 * L0, Dh)
    assert torch.equal(nk[:, :, : Lp + n].cpu().double(), orc.K.view(B, H, -1, Dh)[:, :, : Lp + n].to(dt).double())
    with pytest.raises(RuntimeError, match="must exceed"):
        ffa.grow(10)
    assert ffa.device_status() == 0


@pytest.mark.parametrize("p", [0.0, 1e-3])
def test_pinned_host_inputs_and_output_are_used_in_place(p):
    """q, k, v and out in pinned host memory: no staging copies, the kernels read and write
    them over PCIe.  Same bits as with device tensors."""
    from fastforwardattention_b200 import FastForwardAttn

    dt, B, H, Dh, Lp = torch.float16, 2, 8, 128, 600
    g = torch.Generator().manual_seed(51)
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    a = FastForwardAttn(K.cuda(), V.cuda(), Lp + 3, False)
    b = FastForwardAttn(K.cuda(), V.cuda(), Lp + 3, False)
    qkv = torch.randn(3, 3, B, H, 1, Dh, generator=g).to(dt).pin_memory()      # [step, q/k/v, ...]
    out_h = torch.empty(B, H, Dh, dtype=dt).pin_memory()
    for i in range(3):
        want = a.attention(qkv[i, 0].cuda(), qkv[i, 1].cuda(), qkv[i, 2].cuda(), Dh ** -0.5, Lp + i, p)
        got = b.attention(qkv[i, 0], qkv[i, 1], qkv[i, 2], Dh ** -0.5, Lp + i, p, out=out_h)
        assert got.data_ptr() == out_h.data_ptr()
        torch.cuda.synchronize()
        assert torch.equal(out_h, want.cpu())
    assert torch.equal(a.get_cache()[0], b.get_cache()[0]) and torch.equal(a.get_cache()[1], b.get_cache()[1])
    with pytest.raises(RuntimeError, match="pinned host memory"):
        b.attention(torch.zeros(B, H, 1, Dh, dtype=dt), qkv[0, 1], qkv[0, 2], 0.1, Lp, 0.0)     # pageable: refused
    with pytest.raises(RuntimeError, match="must be contiguous"):
        b.attention(qkv[0, 0].transpose(0, 1), qkv[0, 1], qkv[0, 2], 0.1, Lp, 0.0)
    assert a.device_status() == 0 and b.device_status() == 0
