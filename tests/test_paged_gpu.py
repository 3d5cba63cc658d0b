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


def _unpack_mask(mask: torch.Tensor, rows: int) -> torch.Tensor:
    """[H, words] packed int32 -> [H, rows] bool."""
    m = mask.cpu().to(torch.int64) & 0xFFFFFFFF
    bits = (m[:, :, None] >> torch.arange(32)[None, None, :]) & 1
    return bits.reshape(m.shape[0], -1)[:, :rows].bool()


@pytest.mark.parametrize("path", [1, 2], ids=["cluster-kernel", "streaming-kernel"])
@pytest.mark.parametrize("dt,Dh,pr,max_len", [(torch.float16, 64, 128, 1024), (torch.bfloat16, 128, 256, 1024),
                                              (torch.float32, 80, 128, 1024), (torch.float16, 64, 128, 1152)])
def test_pruned_step_over_pages(dt, Dh, pr, max_len, path):
    """The pruning rule over a paged pool: ragged sequences, pages handed out in a scrambled
    order, a pool poisoned with NaN outside the sequences' rows; kept set and output against
    the restated rule, both kernel paths.  With 1152 rows the fused kernel's slices start
    between page boundaries, so its K tiles arrive as one copy per page."""
    from fastforwardattention_b200 import PagedFastForwardAttn, PagePool

    g = torch.Generator().manual_seed(21 + Dh)
    B, H, Lp = 4, 3, 900
    lengths = [0, pr - 1, pr, 900]
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    pool = PagePool(num_pages=20, heads=H, head_dim=Dh, dtype=dt, device="cuda", page_rows=pr)
    pool._free = [7, 3, 19, 0, 11, 14, 5, 9, 2, 17, 12, 1, 15, 4, 18, 8, 13, 6, 16, 10]
    pool.k.fill_(float("nan"))
    pool.v.fill_(float("nan"))
    seqs = PagedFastForwardAttn(pool, K, V, max_len=max_len, lengths=lengths)
    seqs.engine.set_prune_path(path)
    seqs.engine.record_kept_mask(True)
    Ks = [K[b, :, :lengths[b]] for b in range(B)]
    Vs = [V[b, :, :lengths[b]] for b in range(B)]
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 8e-3}[dt]
    for i, p in enumerate((1e-3, 0.05, 1e-3)):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        q = 2.0 * q
        out = seqs.attention(q.cuda(), k.cuda(), v.cuda(), Dh ** -0.5, p).cpu()
        mask = seqs.engine.get_kept_mask()
        for b in range(B):
            Ks[b] = torch.cat([Ks[b], k[b]], dim=1)
            Vs[b] = torch.cat([Vs[b], v[b]], dim=1)
            rows = lengths[b] + i + 1
            want, kept, info = O.pruned_attention(q[b].view(H, Dh), Ks[b], Vs[b], Dh ** -0.5, p)
            diff = int((_unpack_mask(mask[b], rows) != kept).sum())
            assert diff <= info["borderline"], (b, p, diff, info)
            err = (out[b].double() - want.double()).abs().max().item()
            assert err <= tol + 0.05 * diff, (b, p, err)
    assert seqs.engine.device_status() == 0
    # the appended rows landed in the right pages
    for b in range(B):
        n = lengths[b] + 3
        page = int(seqs.table_host[b, (n - 1) // pr])
        assert torch.equal(pool.k[page, :, (n - 1) % pr].cpu(), Ks[b][:, n - 1])
        assert torch.equal(pool.v[page, :, (n - 1) % pr].cpu(), Vs[b][:, n - 1])


def test_torch_rounding_mode_over_pages():
    """The torch-rounding mode shares the two-pass kernels with pruning; over pages it must
    give what the contiguous engine gives in the same mode."""
    from fastforwardattention_b200 import FastForwardAttn, PagedFastForwardAttn, PagePool

    dt, B, H, Dh, Lp = torch.bfloat16, 2, 4, 128, 700
    g = torch.Generator().manual_seed(10)
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    pool = PagePool(num_pages=16, heads=H, head_dim=Dh, dtype=dt, device="cuda", page_rows=256)
    seqs = PagedFastForwardAttn(pool, K, V, max_len=1024)
    seqs.engine.set_mode("round_like_torch")
    ffa = FastForwardAttn(K.cuda(), V.cuda(), 1024, False)
    ffa.set_mode("round_like_torch")
    for i in range(3):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt).cuda() for _ in range(3))
        a = seqs.attention(q, k, v, Dh ** -0.5)
        b = ffa.attention(q, k, v, Dh ** -0.5, Lp + i, 0)
        assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -9
    assert seqs.engine.device_status() == 0


@pytest.mark.parametrize("dt,Dh,pr", [(torch.float16, 64, 128), (torch.bfloat16, 128, 128), (torch.float32, 80, 128)])
def test_torch_rounding_mode_ragged_over_small_pages(dt, Dh, pr):
    """Every row kept: the cluster kernel streams the V tiles of a slice through its ring.  Ragged
    sequences over 128-row pages handed out in a scrambled order, pool poisoned with NaN outside the
    sequences' rows: tiles that start between page boundaries arrive as one copy per page.  Checked
    against the same-dtype torch function (the mode's target) on every sequence."""
    from fastforwardattention_b200 import PagedFastForwardAttn, PagePool

    g = torch.Generator().manual_seed(5 + Dh)
    B, H, Lp = 4, 3, 900
    lengths = [0, pr - 1, 300, 900]
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    pool = PagePool(num_pages=24, heads=H, head_dim=Dh, dtype=dt, device="cuda", page_rows=pr)
    pool._free = [7, 3, 19, 0, 11, 14, 5, 9, 2, 17, 12, 1, 15, 4, 18, 8, 13, 6, 16, 10, 23, 20, 22, 21]
    pool.k.fill_(float("nan"))
    pool.v.fill_(float("nan"))
    seqs = PagedFastForwardAttn(pool, K, V, max_len=1024, lengths=lengths)
    seqs.engine.set_mode("round_like_torch")
    Ks = [K[b, :, :lengths[b]] for b in range(B)]
    Vs = [V[b, :, :lengths[b]] for b in range(B)]
    gate = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 2e-3}[dt]
    for i in range(3):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        out = seqs.attention(q.cuda(), k.cuda(), v.cuda(), Dh ** -0.5).cpu()
        for b in range(B):
            Ks[b] = torch.cat([Ks[b], k[b]], dim=1)
            Vs[b] = torch.cat([Vs[b], v[b]], dim=1)
            same = O.torch_attn_func(q[b].view(H, 1, Dh), Ks[b], Vs[b], Dh ** -0.5)[:, 0]
            err = (out[b].float() - same.float()).abs().max().item()
            assert err <= gate, (b, i, err)
    assert seqs.engine.device_status() == 0
