"""Paged KV caches: ragged sequences sharing one page pool, against the oracle."""
import pytest
import torch

from oracle import ffa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt,Dh", [(torch.float16, 64), (torch.bfloat16, 128), (torch.float32, 80), (torch.float16, 256)])
def test_ragged_sequences_share_a_pool(dt, Dh):
    from fastforwardattention_b200 import PagedFastForwardAttn, PagePool

    g = torch.Generator().manual_seed(5)
    B, H, Lp, steps, pr = 4, 3, 300, 140, 128
    lengths = [0, 127, 128, 300]                     # empty, just below / on a page boundary, multi-page
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    pool = PagePool(num_pages=24, heads=H, head_dim=Dh, dtype=dt, device="cuda", page_rows=pr)
    pool.k.fill_(float("nan"))                       # anything read outside a sequence's rows poisons the result
    pool.v.fill_(float("nan"))
    seqs = PagedFastForwardAttn(pool, K, V, max_len=512, lengths=lengths)
    assert seqs.pages_in_use == 0 + 1 + 1 + 3 and pool.free_pages == 24 - 5
    # per-sequence oracles (each sequence has its own length)
    orcs = [O.DecodeOracle(K[b:b + 1, :, :lengths[b]], V[b:b + 1, :, :lengths[b]], lengths[b] + steps, compute_dtype=torch.float64)
            for b in range(B)]
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    for i in range(steps):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        out = seqs.attention(q.cuda(), k.cuda(), v.cuda(), Dh ** -0.5)
        if i % 13 == 0 or i == steps - 1:
            for b in range(B):
                ref = orcs[b].step(q[b:b + 1], k[b:b + 1], v[b:b + 1], Dh ** -0.5, lengths[b] + i)
                err = (out[b].cpu().double() - ref[0]).abs().max().item()
                assert err <= tol, (dt, Dh, i, b, err)
        else:
            for b in range(B):
                orcs[b].append(k[b:b + 1], v[b:b + 1], lengths[b] + i)
    # pages were taken only as the sequences grew: ceil((len + steps) / page_rows) each
    want_pages = sum(-(-(n + steps) // pr) for n in lengths)
    assert seqs.pages_in_use == want_pages and pool.free_pages == 24 - want_pages
    assert seqs.engine.device_status() == 0
    seqs.release()
    assert pool.free_pages == 24


def test_paged_matches_contiguous_engine_bitwise_layout_aside():
    """Same inputs through the contiguous engine and through pages handed out in a scrambled
    order: identical outputs (the page indirection changes addresses, not arithmetic)."""
    from fastforwardattention_b200 import FastForwardAttn, PagedFastForwardAttn, PagePool

    dt, B, H, Dh, Lp, steps = torch.bfloat16, 2, 4, 128, 700, 3
    g = torch.Generator().manual_seed(9)
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    pool = PagePool(num_pages=16, heads=H, head_dim=Dh, dtype=dt, device="cuda", page_rows=256)
    pool._free = [3, 11, 0, 7, 14, 5, 9, 2, 12, 1, 15, 4, 8, 13, 6, 10]    # scrambled hand-out order
    seqs = PagedFastForwardAttn(pool, K, V, max_len=1024)
    ffa = FastForwardAttn(K.cuda(), V.cuda(), 1024, False)
    for i in range(steps):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt).cuda() for _ in range(3))
        a = seqs.attention(q, k, v, Dh ** -0.5)
        b = ffa.attention(q, k, v, Dh ** -0.5, Lp + i, 0)
        assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -9
    assert seqs.engine.device_status() == 0 and ffa.device_status() == 0


def test_pool_exhaustion_and_bad_arguments_raise():
    from fastforwardattention_b200 import PagedFastForwardAttn, PagePool

    dt = torch.float16
    with pytest.raises(ValueError, match="multiple of 128"):
        PagePool(4, 2, 64, dt, "cuda", page_rows=100)
    pool = PagePool(num_pages=2, heads=2, head_dim=64, dtype=dt, device="cuda", page_rows=128)
    K = torch.zeros(1, 2, 200, 64, dtype=dt)
    seqs = PagedFastForwardAttn(pool, K, K.clone(), max_len=512)        # takes both pages
    q = torch.zeros(1, 2, 1, 64, dtype=dt, device="cuda")
    for _ in range(56):
        seqs.attention(q, q, q, 0.125)                                   # rows 200..255 fit
    with pytest.raises(MemoryError, match="exhausted"):
        seqs.attention(q, q, q, 0.125)                                   # row 256 needs a third page
    with pytest.raises(MemoryError):
        PagedFastForwardAttn(pool, K, K.clone(), max_len=512)
