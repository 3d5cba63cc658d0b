"""Head-sharded decode on real GPUs: two ranks, one GPU each.  Each rank runs the CUDA engine on
its head shard; local outputs and the all-gathered tensor (fp32: NCCL; fp16: the engine's own
gather over peer memory) are checked against the oracle evaluated on all heads.  Needs two
visible GPUs (skipped otherwise)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from fastforwardattention_b200.sharded import ShardedFastForwardAttn, head_range, shard_heads
        from oracle.ffa_oracle import DecodeOracle

        worst = 0.0
        for dt, tol in ((torch.float16, 2e-3), (torch.float32, 1e-6)):
            g = torch.Generator().manual_seed(3)
            B, H, Dh, Lp, steps = 3, 8, 128, 700, 4
            K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
            V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
            full = DecodeOracle(K, V, Lp + steps)
            eng = ShardedFastForwardAttn(shard_heads(K, rank, world, H).to(dev), shard_heads(V, rank, world, H).to(dev),
                                         Lp + steps, False)
            lo, hi = head_range(H, rank, world)
            peer = dt == torch.float16 and eng.enable_peer_gather()     # fp16: the engine's own gather; fp32: NCCL
            if dt == torch.float16:
                assert peer, "the peer-memory gather could not be set up"
            for i in range(steps):
                q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
                want = full.step(q, k, v, Dh ** -0.5, Lp + i)
                ql, kl, vl = (shard_heads(x, rank, world, H).to(dev) for x in (q, k, v))
                p = 0.0 if i < 3 else 1e-3      # the last step also goes through the pruning kernel
                got = eng.attention(ql, kl, vl, Dh ** -0.5, Lp + i, p, gather=True)
                assert got.shape == (B, H, Dh)
                if p == 0.0:
                    worst = max(worst, (got.cpu().float() - want.float()).abs().max().item() / tol)
                else:
                    assert torch.isfinite(got).all()
            assert eng.engine.device_status() == 0
            eng.close()
        q_out.put((rank, worst))
    finally:
        dist.destroy_process_group()


def test_two_ranks_nccl_gather_matches_oracle():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(w <= 1.0 for _, w in res), res     # error / tolerance


def _graph_worker(rank, world, port, q_out):
    """Each rank records ONE graph holding its attention step and the peer-memory gather and
    replays it for every token: the row index and the gather's step number both live in
    device memory."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from fastforwardattention_b200.sharded import ShardedFastForwardAttn, shard_heads
        from oracle.ffa_oracle import DecodeOracle

        dt, tol = torch.bfloat16, 8e-3
        g = torch.Generator().manual_seed(6)
        B, H, Dh, Lp, steps = 2, 8, 128, 300, 5
        Hl = H // world
        K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
        V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
        full = DecodeOracle(K, V, Lp + steps + 1, compute_dtype=torch.float64)
        sh = ShardedFastForwardAttn(shard_heads(K, rank, world, H).to(dev), shard_heads(V, rank, world, H).to(dev),
                                    Lp + steps + 1, False)
        assert sh.enable_peer_gather()
        eng = sh.engine
        q_s, k_s, v_s = (torch.zeros(B, Hl, 1, Dh, dtype=dt, device=dev) for _ in range(3))
        local = torch.zeros(B, Hl, Dh, dtype=dt, device=dev)
        gathered = torch.zeros(B, H, Dh, dtype=dt, device=dev)
        rows = torch.full((B,), Lp, dtype=torch.int32, device=dev)

        def step():
            eng.attention_per_sample(q_s, k_s, v_s, Dh ** -0.5, rows, 0.0, out=local)
            eng.peer_gather(local, out=gathered)
            rows.add_(1)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()                                   # eager warm-up = token 0 (inputs are zeros on every rank)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        z = torch.zeros(B, H, 1, Dh, dtype=dt)
        full.step(z, z, z, Dh ** -0.5, Lp)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            step()
        worst = 0.0
        for i in range(1, steps + 1):
            q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
            for dst, src in ((q_s, q), (k_s, k), (v_s, v)):
                dst.copy_(shard_heads(src, rank, world, H))
            graph.replay()
            want = full.step(q, k, v, Dh ** -0.5, Lp + i)
            worst = max(worst, (gathered.cpu().double() - want).abs().max().item() / tol)
        assert eng.device_status() == 0
        sh.close()
        q_out.put((rank, worst))
    finally:
        dist.destroy_process_group()


def test_two_ranks_step_and_gather_replayed_from_one_graph_per_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_graph_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(w <= 1.0 for _, w in res), res


def _host_step_worker(rank, world, port, q_out):
    """ShardedFastForwardAttn.graphed_step(): upload of the rank's q/k/v slice from pinned host memory, then one graph
    with the attention launch, the peer-memory gather and the download of the full [B, H, Dh] result."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from fastforwardattention_b200.sharded import ShardedFastForwardAttn, shard_heads
        from oracle.ffa_oracle import DecodeOracle

        dt, tol = torch.float16, 2e-3
        g = torch.Generator().manual_seed(8)
        B, H, Dh, Lp, steps = 2, 8, 64, 260, 5
        K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
        V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
        full = DecodeOracle(K, V, Lp + steps, compute_dtype=torch.float64)
        sh = ShardedFastForwardAttn(shard_heads(K, rank, world, H).to(dev), shard_heads(V, rank, world, H).to(dev),
                                    Lp + steps, False)
        assert sh.enable_peer_gather()
        step = sh.graphed_step(Dh ** -0.5, first_row=Lp)
        worst = 0.0
        for i in range(steps):
            qkv = torch.randn(3, B, H, 1, Dh, generator=g).to(dt)
            mine = torch.stack([shard_heads(qkv[j], rank, world, H) for j in range(3)]).pin_memory()
            out = step(mine)
            torch.cuda.current_stream(dev).synchronize()
            assert out.shape == (B, H, Dh)
            want = full.step(qkv[0], qkv[1], qkv[2], Dh ** -0.5, Lp + i)
            worst = max(worst, (out.double() - want).abs().max().item() / tol)
        assert sh.engine.device_status() == 0
        sh.close()
        q_out.put((rank, worst))
    finally:
        dist.destroy_process_group()


def test_two_ranks_graphed_host_step():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_host_step_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(w <= 1.0 for _, w in res), res
