"""The peer-memory all-gather of the step outputs, with all ranks emulated on ONE GPU.

The ranks of a node normally are processes on different GPUs.  Here the engines of all ranks
live in one process and share one stream, and the two phases of the gather are issued
separately -- every rank's push, then every rank's wait -- so that no kernel ever waits for a
kernel queued behind it.  The buffers are attached by raw pointer (same process, no handles).
"""
import pytest
import torch

from oracle import ffa_oracle as O

pytestmark = pytest.mark.gpu


def _ranks(world, dt, B, H, Dh, Lp, max_len, g):
    from fastforwardattention_b200 import FastForwardAttn

    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    per = H // world
    engines = [FastForwardAttn(K[:, r * per:(r + 1) * per].contiguous().cuda(), V[:, r * per:(r + 1) * per].contiguous().cuda(),
                               max_len, False) for r in range(world)]
    for e in engines:
        assert len(bytes(e.peer_gather_alloc(world))) == 64
    ptrs = [e.peer_gather_ptr() for e in engines]
    for r, e in enumerate(engines):
        e.peer_gather_attach(world, r, ptrs, False)
    return K, V, engines


@pytest.mark.parametrize("world,dt,Dh,H", [(2, torch.bfloat16, 128, 4), (4, torch.float32, 80, 8), (8, torch.float16, 64, 8)])
def test_every_rank_receives_every_slice(world, dt, Dh, H):
    g = torch.Generator().manual_seed(40 + world)
    B, Lp, steps = 3, 150, 5
    per = H // world
    K, V, engines = _ranks(world, dt, B, H, Dh, Lp, Lp + steps, g)
    orc = O.DecodeOracle(K, V, Lp + steps, compute_dtype=torch.float64)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    for i in range(steps):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        outs = [e.attention(q[:, r * per:(r + 1) * per].contiguous().cuda(), k[:, r * per:(r + 1) * per].contiguous().cuda(),
                            v[:, r * per:(r + 1) * per].contiguous().cuda(), Dh ** -0.5, Lp + i, 1e-3 if i == 3 else 0.0)
                for r, e in enumerate(engines)]
        got = [e.peer_gather(o, phases=1) for e, o in zip(engines, outs)]          # all pushes ...
        got = [e.peer_gather(o, phases=2, out=x) for e, o, x in zip(engines, outs, got)]   # ... before any wait
        want = torch.cat(outs, dim=1)                  # rank-major heads
        for r in range(world):
            assert got[r].shape == (B, H, Dh)
            assert torch.equal(got[r], want), (i, r)
        if i != 3:
            ref = orc.step(q, k, v, Dh ** -0.5, Lp + i)
            assert (got[0].cpu().double() - ref).abs().max().item() <= tol
        else:
            orc.append(k, v, Lp + i)
    assert all(e.device_status() == 0 for e in engines)
    for e in engines:
        e.peer_gather_free()


@pytest.mark.parametrize("world,dt,B,H,Dh,Lp,cluster_merge",
                         [(4, torch.float16, 40, 32, 64, 100, True),      # 320 pairs per rank: CTAs of whole pairs
                          (2, torch.bfloat16, 3, 4, 128, 150, True),      # few pairs: a thread-block cluster per pair, its leader writes
                          (2, torch.bfloat16, 3, 4, 128, 150, False),     # the same cut, merged through global memory by the last arriver
                          (2, torch.float32, 1, 2, 64, 20000, True),      # one pair per rank over several clusters: the leaders' last arriver
                          (8, torch.float16, 2, 8, 80, 300, True)])
def test_attention_kernel_pushes_its_rows_and_a_short_kernel_collects(world, dt, B, H, Dh, Lp, cluster_merge):
    """The fused form of the gather: the exact kernel's epilogue stores every output row into the peers' staging buffers
    (and the own result) as it produces it and raises the flags after the step's last pair; only the wait-and-collect
    kernel follows.  Pruned steps in between do not push and take the whole gather kernel."""
    g = torch.Generator().manual_seed(50 + world)
    steps, per = 4, H // world
    K, V, engines = _ranks(world, dt, B, H, Dh, Lp, Lp + steps, g)
    orc = O.DecodeOracle(K, V, Lp + steps, compute_dtype=torch.float64)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    full = [torch.zeros(B, H, Dh, dtype=dt, device="cuda") for _ in engines]
    for e, f in zip(engines, full):
        e.set_cluster_merge(cluster_merge)
        e.set_push_target(f)
    sl = lambda x, r: x[:, r * per:(r + 1) * per].contiguous().cuda()
    for i in range(steps):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        p = 1e-3 if i == 2 else 0.0
        outs = [e.attention(sl(q, r), sl(k, r), sl(v, r), Dh ** -0.5, Lp + i, p) for r, e in enumerate(engines)]   # exact steps push here
        if p > 0:
            for e, o, f in zip(engines, outs, full):
                e.peer_gather(o, phases=1, out=f)
        got = [e.peer_gather(o, phases=2, out=f) for e, o, f in zip(engines, outs, full)]
        want = torch.cat(outs, dim=1)
        for r in range(world):
            assert torch.equal(got[r], want), (i, r)
        if p == 0:
            ref = orc.step(q, k, v, Dh ** -0.5, Lp + i)
            assert (got[0].cpu().double() - ref).abs().max().item() <= tol
        else:
            orc.append(k, v, Lp + i)
    assert all(e.device_status() == 0 for e in engines)
    for e in engines:
        e.set_push_target(None)
        e.peer_gather_free()


def test_wait_for_a_silent_peer_runs_out_and_reports():
    """Rank 1 never pushes: rank 0's wait gives up after its limit, the time-out bit appears in
    the status word, the context stays usable, and the pair recovers on the next step."""
    import time

    g = torch.Generator().manual_seed(44)
    dt, B, H, Dh, Lp = torch.float16, 2, 4, 64, 40
    K, V, (e0, e1) = _ranks(2, dt, B, H, Dh, Lp, Lp + 2, g)
    q = torch.randn(B, 2, 1, Dh, generator=g).to(dt).cuda()
    o0 = e0.attention(q, q, q, 0.125, Lp, 0.0)
    torch.cuda.synchronize()
    t0 = time.time()
    e0.peer_gather(o0, phases=3, wait_limit_ms=100)
    assert e0.device_status() == 1                    # synchronises; FFA_STATUS_WAIT_TIMEOUT
    assert 0.09 <= time.time() - t0 < 1.5
    assert e0.device_status() == 0                    # reading the word clears it
    # rank 1 catches up with the same step, then both do one more
    o1 = e1.attention(q, q, q, 0.125, Lp, 0.0)
    e1.peer_gather(o1, phases=3, wait_limit_ms=100)    # rank 0's flag is already there
    for t in (Lp + 1,):
        o0, o1 = e0.attention(q, q, q, 0.125, t, 0.0), e1.attention(q, q, q, 0.125, t, 0.0)
        g0, g1 = e0.peer_gather(o0, phases=1), e1.peer_gather(o1, phases=1)
        g0, g1 = e0.peer_gather(o0, phases=2, out=g0), e1.peer_gather(o1, phases=2, out=g1)
        assert torch.equal(g0, torch.cat([o0, o1], dim=1)) and torch.equal(g1, g0)
    assert e0.device_status() == 0 and e1.device_status() == 0


def test_bad_arguments_raise():
    from fastforwardattention_b200 import FastForwardAttn

    dt = torch.float16
    K = torch.zeros(1, 2, 8, 64, dtype=dt, device="cuda")
    e = FastForwardAttn(K, K.clone(), 16, False)
    with pytest.raises(RuntimeError, match="peer_gather_attach first"):
        e.peer_gather(torch.zeros(1, 2, 64, dtype=dt, device="cuda"))
    with pytest.raises(RuntimeError, match="outside"):
        e.peer_gather_alloc(9)
    e.peer_gather_alloc(2)
    with pytest.raises(RuntimeError, match="already allocated"):
        e.peer_gather_alloc(2)
    with pytest.raises(RuntimeError, match="own buffer"):
        e.peer_gather_attach(2, 0, [e.peer_gather_ptr() + 256, e.peer_gather_ptr()], False)
    with pytest.raises(RuntimeError, match="one buffer pointer per rank"):
        e.peer_gather_attach(2, 2, [e.peer_gather_ptr(), e.peer_gather_ptr()], False)
    e.peer_gather_attach(1, 0, [e.peer_gather_ptr()], False)
    o = torch.ones(1, 2, 64, dtype=dt, device="cuda")
    with pytest.raises(RuntimeError, match="wait_limit_ms"):
        e.peer_gather(o, 3, 5000)
    with pytest.raises(RuntimeError, match="phases"):
        e.peer_gather(o, 0, 100)
    assert torch.equal(e.peer_gather(o), o)           # a world of one gathers its own slice
    e.peer_gather_free()


def test_gather_replayed_from_a_cuda_graph():
    """The step number lives in device memory, so a push and a wait recorded once can be
    replayed for every step (two ranks on one GPU: one graph holds both pushes, then both
    waits)."""
    g = torch.Generator().manual_seed(45)
    dt, B, H, Dh, Lp = torch.bfloat16, 2, 4, 128, 30
    K, V, (e0, e1) = _ranks(2, dt, B, H, Dh, Lp, Lp + 1, g)
    o0 = torch.zeros(B, 2, Dh, dtype=dt, device="cuda")
    o1 = torch.zeros_like(o0)
    g0 = torch.zeros(B, H, Dh, dtype=dt, device="cuda")
    g1 = torch.zeros_like(g0)

    def both():
        e0.peer_gather(o0, phases=1, out=g0), e1.peer_gather(o1, phases=1, out=g1)
        e0.peer_gather(o0, phases=2, out=g0), e1.peer_gather(o1, phases=2, out=g1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        both()                                         # step 1, eagerly
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        both()
    for step in range(5):                              # steps 2..6 from the graph: both halves, flags growing
        o0.copy_(torch.randn(B, 2, Dh, generator=g).to(dt))
        o1.copy_(torch.randn(B, 2, Dh, generator=g).to(dt))
        graph.replay()
        want = torch.cat([o0, o1], dim=1)
        assert torch.equal(g0, want) and torch.equal(g1, want), step
    assert e0.device_status() == 0 and e1.device_status() == 0
