"""Host logic of the head-sharded path on two CPU ranks (gloo).  The per-rank engine is a
stand-in built on the oracle: what is tested here is the partition arithmetic and the
gather layout, not the kernel."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class OracleEngine:
    def __init__(self, K, V, max_len, use_default):
        from oracle.ffa_oracle import DecodeOracle

        self.o = DecodeOracle(K, V, max_len)

    def attention(self, q, k, v, scale, t, p=0.0):
        return self.o.step(q, k, v, scale, t)

    def get_cache(self):
        return self.o.K, self.o.V


def _worker(rank, world, port, q_out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fastforwardattention_b200.sharded import ShardedFastForwardAttn, head_range, shard_heads
        from oracle.ffa_oracle import DecodeOracle

        g = torch.Generator().manual_seed(0)
        B, H, Dh, Lp, steps = 2, 4, 64, 9, 3
        K = torch.randn(B, H, Lp, Dh, generator=g)
        V = torch.randn(B, H, Lp, Dh, generator=g)
        full = DecodeOracle(K, V, Lp + steps)
        eng = ShardedFastForwardAttn(shard_heads(K, rank, world, H), shard_heads(V, rank, world, H), Lp + steps,
                                     False, engine_factory=OracleEngine)
        assert head_range(H, rank, world) == (rank * H // world, (rank + 1) * H // world)
        worst = 0.0
        for i in range(steps):
            q, k, v = (torch.randn(B, 1, H * Dh, generator=g) for _ in range(3))   # HF layout
            want = full.step(q, k, v, 0.125, Lp + i)
            ql, kl, vl = (shard_heads(x, rank, world, H) for x in (q, k, v))
            local = eng.attention(ql, kl, vl, 0.125, Lp + i)
            lo, hi = head_range(H, rank, world)
            worst = max(worst, (local - want[:, lo:hi]).abs().max().item())
            got = eng.attention(ql, kl, vl, 0.125, Lp + i, gather=True)
            assert got.shape == (B, H, Dh)
            worst = max(worst, (got - want).abs().max().item())
        q_out.put((rank, worst))
    finally:
        dist.destroy_process_group()


def test_head_sharding_and_gather_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(w < 1e-6 for _, w in res)


def test_head_range_rejects_uneven_split():
    from fastforwardattention_b200.sharded import head_range

    with pytest.raises(ValueError):
        head_range(6, 0, 4)


def _worker_peer_leaves(rank, world, port, q_out):
    """Rank 1 leaves between steps; rank 0 must get an error from the next gather, not a hang."""
    import datetime
    import time

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from fastforwardattention_b200.sharded import ShardedFastForwardAttn, shard_heads

    g = torch.Generator().manual_seed(1)
    B, H, Dh, Lp = 1, 4, 64, 5
    K = torch.randn(B, H, Lp, Dh, generator=g)
    V = torch.randn(B, H, Lp, Dh, generator=g)
    eng = ShardedFastForwardAttn(shard_heads(K, rank, world, H), shard_heads(V, rank, world, H), Lp + 2, False,
                                 engine_factory=OracleEngine)
    q, k, v = (shard_heads(torch.randn(B, H, 1, Dh, generator=g), rank, world, H) for _ in range(3))
    full = eng.attention(q, k, v, 0.125, Lp, gather=True)          # step 0: everybody is there
    assert full.shape == (B, H, Dh)
    def report(msg):
        q_out.put((rank, msg))
        q_out.close()
        q_out.join_thread()                                        # flushed before the process goes away
        os._exit(0)

    if rank == 1:
        report("left")                                             # leaves between steps, nothing in flight
    t0 = time.time()
    try:
        eng.attention(q, k, v, 0.125, Lp + 1, gather=True)         # step 1: the peer is gone
        report("no error")
    except Exception as e:                                         # noqa: BLE001 - any backend error type
        report(f"error after {time.time() - t0:.1f}s: {type(e).__name__}")


def test_gather_fails_instead_of_hanging_when_a_rank_leaves():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_peer_leaves, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(30)
    assert res[1] == "left"
    assert res[0].startswith("error after"), res


class PeerStandIn(OracleEngine):
    """OracleEngine plus the peer-gather surface of the extension class.  Memory cannot be shared
    between CPU ranks here, so peer_gather itself goes through the group; what the test checks
    is the set-up protocol around it."""
    fail_on_rank = -1

    def __init__(self, K, V, max_len, use_default):
        super().__init__(K, V, max_len, use_default)
        self.rank = dist.get_rank()
        self.log = []

    def peer_gather_alloc(self, world):
        if self.rank == self.fail_on_rank:
            raise RuntimeError("no memory for the peer buffer")
        self.log.append(("alloc", world))
        return bytes([self.rank]) * 64

    def peer_gather_ptr(self):
        return 1000 + self.rank

    def peer_mem_open(self, handle):
        assert len(handle) == 64 and len(set(handle)) == 1
        self.log.append(("open", handle[0]))
        return 2000 + handle[0]

    def peer_mem_close(self, ptr):
        self.log.append(("close", ptr))

    def peer_gather_attach(self, world, rank, ptrs, close_on_free):
        self.log.append(("attach", world, rank, tuple(ptrs), close_on_free))

    def peer_gather(self, out_local):
        self.log.append(("gather",))
        parts = [torch.empty_like(out_local) for _ in range(dist.get_world_size())]
        dist.all_gather(parts, out_local)
        return torch.cat(parts, dim=1)

    def attention(self, q, k, v, scale, t, p=0.0, gather_into=None):
        out = super().attention(q, k, v, scale, t, p)
        if gather_into is None:
            return out
        gather_into.copy_(self.peer_gather(out))     # the extension pushes from the attention kernel, then collects
        return gather_into

    def peer_gather_detach(self):
        self.log.append(("detach",))

    def peer_gather_free(self):
        self.log.append(("free",))


def _peer_worker(rank, world, port, q_out, fail_on_rank):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fastforwardattention_b200.sharded import ShardedFastForwardAttn, shard_heads
        from oracle.ffa_oracle import DecodeOracle

        PeerStandIn.fail_on_rank = fail_on_rank
        g = torch.Generator().manual_seed(1)
        B, H, Dh, Lp = 2, 4, 64, 5
        K = torch.randn(B, H, Lp, Dh, generator=g)
        V = torch.randn(B, H, Lp, Dh, generator=g)
        full = DecodeOracle(K, V, Lp + 1)
        eng = ShardedFastForwardAttn(shard_heads(K, rank, world, H), shard_heads(V, rank, world, H), Lp + 1,
                                     False, engine_factory=PeerStandIn)
        enabled = eng.enable_peer_gather()
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g) for _ in range(3))
        want = full.step(q, k, v, 0.125, Lp)
        got = eng.attention(*(shard_heads(x, rank, world, H) for x in (q, k, v)), 0.125, Lp, gather=True)
        err = (got - want).abs().max().item()
        eng.close()
        q_out.put((rank, enabled, err, eng.engine.log))
        q_out.close()
        q_out.join_thread()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_on_rank", [-1, 1])
def test_peer_gather_setup_protocol(fail_on_rank):
    """Every rank maps every other rank's buffer, in rank order, with its own pointer in its own
    place; if one rank cannot set up, all ranks fall back to the process group together."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, q, fail_on_rank)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, enabled, err, log in res:
        assert err < 1e-6
        other = 1 - rank
        if fail_on_rank < 0:
            assert enabled
            want_ptrs = (1000, 2001) if rank == 0 else (2000, 1001)
            assert log == [("alloc", 2), ("open", other), ("attach", 2, rank, want_ptrs, True), ("gather",), ("detach",), ("free",)]
        else:
            assert not enabled
            assert ("gather",) not in log and not any(e[0] == "attach" for e in log)
            if rank != fail_on_rank:
                assert log[0] == ("alloc", 2) and log[-1] == ("free",)     # its own buffer is released again
