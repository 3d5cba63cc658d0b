"""CPU tests of the oracle itself: pinned against the golden vectors (outputs of the
reference's own function text) and against the CUDA toolkit's host evaluation of the fp16
comparison used by the reference's pruning rule."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import ffa_oracle as O
from tests.helpers import golden_names, load_golden

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", golden_names())
def test_oracle_reproduces_golden(name):
    g = load_golden(name)
    torch.set_num_threads(1)  # the fixtures were generated single-threaded
    orc = O.DecodeOracle(g["K"], g["V"], g["prompt"] + len(g["steps"]))
    for i, (q, k, v, want) in enumerate(g["steps"]):
        got = orc.step(q, k, v, g["scale"], g["prompt"] + i)
        # same operands, same torch kernels: bit-exact on the machine that made the fixtures;
        # one unit in the last place of the dtype is allowed for a different CPU's bmm kernels
        ulp = {torch.float32: 2e-7, torch.float16: 1e-3, torch.bfloat16: 8e-3}[g["dtype"]]
        err = (got.float() - want.float()).abs().max().item()
        assert err <= ulp * max(1.0, want.float().abs().max().item()), (name, i, err)


@pytest.mark.parametrize("name", golden_names())
def test_upcast_reference_is_close_to_golden(name):
    g = load_golden(name)
    B, H, Lp, Dh = g["K"].shape
    orc = O.DecodeOracle(g["K"], g["V"], Lp + len(g["steps"]), compute_dtype=torch.float64)
    for i, (q, k, v, want) in enumerate(g["steps"]):
        got = orc.step(q, k, v, g["scale"], Lp + i)
        tol = {torch.float32: 2e-6, torch.float16: 4e-3, torch.bfloat16: 6e-2}[g["dtype"]]
        assert (got.float() - want.float()).abs().max().item() < tol


def _leq_lib():
    so = os.path.join(ROOT, "oracle", "_build", "libhalf_leq_host.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "host"], check=True, capture_output=True)
    return ctypes.CDLL(so)


def test_fp16_leq_restatement_matches_toolkit_host_code():
    """All 65536 patterns through the numeric constructor, and the comparison on every pair
    (a, b) with b on a grid plus the neighbours of a -- the reference expression
    `__hle(uint16_t, uint16_t)` (attention.cu:466-469) evaluated by cuda_fp16.h on the host."""
    lib = _leq_lib()
    a = np.arange(65536, dtype=np.uint16)
    out = np.zeros(65536, dtype=np.uint16)
    lib.ffa_ref_half_from_bits_numeric(a.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                       ctypes.c_size_t(a.size))
    mine = O.half_bits_as_number_rn(a).view(np.uint16)
    assert np.array_equal(out, mine)

    rng = np.random.default_rng(0)
    aa = np.concatenate([a, a, a, rng.integers(0, 0x3C01, 1 << 20).astype(np.uint16)])
    bb = np.concatenate([np.clip(a.astype(np.int32) - 1, 0, 65535).astype(np.uint16), a,
                         np.clip(a.astype(np.int32) + 1, 0, 65535).astype(np.uint16),
                         rng.integers(0, 0x3C01, 1 << 20).astype(np.uint16)])
    res = np.zeros(aa.size, dtype=np.uint8)
    lib.ffa_ref_half_leq(aa.ctypes.data_as(ctypes.c_void_p), bb.ctypes.data_as(ctypes.c_void_p),
                         res.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(aa.size))
    ta = torch.from_numpy(aa.view(np.int16).copy()).view(torch.float16)
    tb = torch.from_numpy(bb.view(np.int16).copy()).view(torch.float16)
    got = O.leq_reference(ta, tb).numpy().astype(np.uint8)
    assert np.array_equal(res, got)
    # the documented quirk: one ulp above still compares "<=" once patterns exceed 2048
    assert O.leq_reference(torch.tensor([0x1C02], dtype=torch.int16).view(torch.float16),
                           torch.tensor([0x1C01], dtype=torch.int16).view(torch.float16)).item()
    assert not O.leq_reference(torch.tensor([0x0401], dtype=torch.int16).view(torch.float16),
                               torch.tensor([0x0400], dtype=torch.int16).view(torch.float16)).item()


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_pruning_rule_p0_is_exact_attention(dt):
    g = torch.Generator().manual_seed(5)
    N, L, Dh = 6, 50, 64
    q = torch.randn(N, Dh, generator=g).to(dt)
    K = torch.randn(N, L, Dh, generator=g).to(dt)
    V = torch.randn(N, L, Dh, generator=g).to(dt)
    out, kept, info = O.pruned_attention(q, K, V, 0.125, 0.0, eps=0.0)
    ref = O.attention_reference(q[:, None], K, V, 0.125, torch.float64)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dt]
    assert (out.double() - ref).abs().max().item() < tol
    assert kept[:, -1].all()


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_pruning_rule_semantics(dt):
    """Threshold is a fraction of the max probability, the new token is never pruned, masked
    keys are never kept, probabilities are not renormalised."""
    g = torch.Generator().manual_seed(6)
    N, L, Dh = 4, 200, 64
    q = torch.randn(N, Dh, generator=g)
    K = 0.5 * torch.randn(N, L, Dh, generator=g)
    peaks = torch.rand(N, L, generator=g) < 0.05
    peaks[:, 3] = True
    K = torch.where(peaks[..., None], 4 * q[:, None, :], K)
    K[:, -1] = 0.0  # new token gets a hopeless score: must still be kept
    V = torch.randn(N, L, Dh, generator=g)
    q, K, V = q.to(dt), K.to(dt), V.to(dt)
    fk = torch.tensor([0, 5, 0, 17], dtype=torch.int32)
    out, kept, info = O.pruned_attention(q, K, V, 0.125, 1e-3, first_key=fk)
    assert kept[:, -1].all()
    for n in range(N):
        assert not kept[n, : fk[n]].any()
        assert torch.equal(kept[n, fk[n]:-1], peaks[n, fk[n]:-1])
    assert info["borderline"] == 0
    s = torch.einsum("nd,nld->nl", q.float(), K.float()) * 0.125
    s = s.masked_fill(torch.arange(L)[None] < fk[:, None], -float("inf"))
    Pfull = torch.softmax(s, -1)
    want = torch.einsum("nl,nld->nd", Pfull * kept, V.float())
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dt]
    assert (out.float() - want).abs().max().item() < tol


def test_rounding_points_restatement_tracks_same_dtype_torch():
    g = torch.Generator().manual_seed(8)
    for dt, tol in ((torch.float16, 3e-4), (torch.bfloat16, 2e-3)):
        N, L, Dh = 64, 512, 128
        q = torch.randn(N, Dh, generator=g).to(dt)
        K = torch.randn(N, L, Dh, generator=g).to(dt)
        V = torch.randn(N, L, Dh, generator=g).to(dt)
        same = O.torch_attn_func(q[:, None], K, V, Dh ** -0.5)[:, 0]
        mine = O.torch_rounding_points(q, K, V, Dh ** -0.5)
        assert (same.float() - mine.float()).abs().max().item() <= tol
