"""Seeded random configurations through the C ABI against the oracle: dtypes, head dims,
batch/head counts, cache lengths, the three length modes, pruning on both paths, random launch
shapes.  Small sizes, many combinations."""
import random

import pytest
import torch

from fastforwardattention_b200 import capi
from oracle import ffa_oracle as O
from tests.cabi_engine import CAbiEngine

pytestmark = pytest.mark.gpu

DTS = [torch.float32, torch.float16, torch.bfloat16]


def oracle_step(q, Kc, Vc, k, v, scale, rows, first, p, dt):
    """Per-sample reference: sample b attends rows [first[b], rows[b]) of the cache plus the new token."""
    B, H, Dh = q.shape[0], q.shape[1], q.shape[-1]
    outs, kepts, border = [], [], 0
    for b in range(B):
        L = int(rows[b])
        Kb = torch.cat([Kc[b, :, :L], k[b]], dim=1)
        Vb = torch.cat([Vc[b, :, :L], v[b]], dim=1)
        fk = torch.full((H,), int(first[b]), dtype=torch.int32)
        o, kept, info = O.pruned_attention(q[b, :, 0], Kb, Vb, scale, p, first_key=fk, eps=1e-6 if p > 0 else 0.0)
        outs.append(o), kepts.append(kept)
        border += info["borderline"]
    return outs, kepts, border


@pytest.mark.parametrize("seed", range(48))
def test_random_configuration(seed):
    rng = random.Random(seed)
    dt = rng.choice(DTS)
    Dh = rng.choice([64, 80, 128, 256])
    B, H = rng.randint(1, 5), rng.randint(1, 6)
    Lmax = rng.choice([1, 2, 9, 33, 100, 257, 700, 1300])
    run_random_steps(seed, rng, dt, Dh, B, H, Lmax, force_launch=rng.random() < 0.6)


@pytest.mark.parametrize("seed", range(100, 116))
def test_random_few_pairs_long_caches(seed):
    """One to eight (batch, head) pairs over thousands of rows, planner's own launch shape: a pair
    is spread over one or several thread-block clusters, in all three length modes."""
    rng = random.Random(seed)
    dt = rng.choice(DTS)
    Dh = rng.choice([64, 80, 128, 256])
    B, H = rng.randint(1, 2), rng.randint(1, 4)
    Lmax = rng.choice([3000, 9000, 20000])
    run_random_steps(seed, rng, dt, Dh, B, H, Lmax, force_launch=False)


def run_random_steps(seed, rng, dt, Dh, B, H, Lmax, force_launch):
    mode = rng.choice(["uniform", "left", "per_sample"])
    p = rng.choice([0.0, 0.0, 1e-3, 0.05])
    path = rng.choice([0, 1, 2])
    g = torch.Generator().manual_seed(1000 + seed)
    Kc = torch.randn(B, H, Lmax, Dh, generator=g).to(dt)
    Vc = torch.randn(B, H, Lmax, Dh, generator=g).to(dt)
    eng = CAbiEngine(Kc, Vc, Lmax)     # whole cache pre-filled; steps overwrite their row
    eng.set_prune_path(path)
    if force_launch:
        eng.set_launch(tile_rows=rng.choice([8, 16, 32, 64]), stages=rng.choice([2, 3, 4]),
                       consumer_warps=rng.choice([1, 2, 4, 8]), ctas_per_sm=rng.choice([1, 2, 4]),
                       grid=rng.choice([0, 0, 1, 7]))
    scale = Dh ** -0.5
    for step in range(2):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        q = 1.5 * q
        t = rng.randint(0, Lmax - 1)
        if mode == "uniform":
            rows, first = [t] * B, [0] * B
            got = eng.attention(q, k, v, scale, t, p=p, want_mask=p > 0)
        elif mode == "left":
            rows, first = [t] * B, [rng.randint(0, t) for _ in range(B)]
            got = eng.attention(q, k, v, scale, t, p=p, seq_lengths=torch.tensor(first, dtype=torch.int32),
                                right_or_no_padding=False, want_mask=p > 0)
        else:
            rows, first = [rng.randint(0, Lmax - 1) for _ in range(B)], [0] * B
            bound = rng.choice([max(rows), Lmax - 1])   # what the host knows about the lengths: tight or nothing
            got = eng.attention(q, k, v, scale, bound, p=p, seq_lengths=torch.tensor(rows, dtype=torch.int32),
                                right_or_no_padding=True, want_mask=p > 0)
        outs, kepts, border = oracle_step(q, Kc, Vc, k, v, scale, rows, first, p, dt)
        tol = {torch.float32: 2e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dt]
        ndiff = 0
        for b in range(B):
            if p > 0:
                L = rows[b]
                mine = eng.kept(L)[b * H:(b + 1) * H, : L + 1]
                ndiff += int((mine != kepts[b]).sum())
        assert ndiff <= border, (seed, "kept sets", ndiff, border)
        for b in range(B):
            err = (got[b].cpu().float() - outs[b].float()).abs().max().item()
            assert err <= tol + 0.3 * ndiff, (seed, dt, Dh, B, H, Lmax, mode, p, path, step, b, err)
            # the step wrote its row and nothing else moved
            Kc[b, :, rows[b]] = k[b, :, 0]
            Vc[b, :, rows[b]] = v[b, :, 0]
        assert torch.equal(eng.k_cache.cpu(), Kc) and torch.equal(eng.v_cache.cpu(), Vc), (seed, "cache contents")
    assert eng.status() == 0


@pytest.mark.parametrize("seed", range(300, 332))
def test_random_torch_rounding_mode(seed):
    """The torch-rounding mode on random shapes against its target, the same-dtype torch function:
    fp32 within 2e-6, fp16 and bf16 within 2e-3; with and without a score scratch bound (the
    scores stay in shared memory), planner's choice or the cluster kernel forced."""
    rng = random.Random(seed)
    dt = rng.choice(DTS)
    Dh = rng.choice([64, 80, 128, 256])
    B, H = rng.randint(1, 4), rng.randint(1, 6)
    Lmax = rng.choice([1, 2, 9, 33, 100, 257, 700, 1300, 2100, 5000])
    g = torch.Generator().manual_seed(5000 + seed)
    Kc = torch.randn(B, H, Lmax, Dh, generator=g).to(dt)
    Vc = torch.randn(B, H, Lmax, Dh, generator=g).to(dt)
    eng = CAbiEngine(Kc, Vc, Lmax, with_scores=rng.random() < 0.5)
    eng.set_mode(1)
    eng.set_prune_path(rng.choice([0, 0, 1]))
    scale = Dh ** -0.5
    gate = {torch.float32: 2e-6, torch.float16: 2e-3, torch.bfloat16: 2e-3}[dt]
    for step in range(2):
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt) for _ in range(3))
        t = rng.randint(0, Lmax - 1)
        got = eng.attention(q, k, v, scale, t).cpu()
        Kc[:, :, t] = k[:, :, 0]
        Vc[:, :, t] = v[:, :, 0]
        same = O.torch_attn_func(q.reshape(B * H, 1, Dh), Kc[:, :, :t + 1].reshape(B * H, t + 1, Dh),
                                 Vc[:, :, :t + 1].reshape(B * H, t + 1, Dh), scale)[:, 0].reshape(B, H, Dh)
        err = (got.float() - same.float()).abs().max().item()
        assert err <= gate, (seed, dt, Dh, B, H, Lmax, t, err)
        assert torch.equal(eng.k_cache.cpu(), Kc) and torch.equal(eng.v_cache.cpu(), Vc), (seed, "cache contents")
    assert eng.status() == 0
