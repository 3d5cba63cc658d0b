"""The workspace-free entry point, ffa_attention_static_scratch.

Some hosts cannot give the engine scratch memory at call time (their allocator already owns
the whole GPU, or their decode thread may not take cudaMalloc's device-wide synchronisation,
or they are a plain C caller holding only the tensors of the call).  For them the library
keeps the scratch in a static device array.  This test drives that entry point through the C
ABI next to the regular one on identical inputs, two steps in a row (the second step sees
the scratch exactly as the first left it), and checks the size limit is enforced.

Collected last on purpose: a failure here must not hide results of the other GPU tests.
"""
import ctypes as C
import math

import pytest
import torch

from fastforwardattention_b200 import capi
from oracle import ffa_oracle as O
from tests.cabi_engine import CODE, CAbiEngine, _ptr, _stream
from tests.helpers import TOL, assert_close_ulp

pytestmark = pytest.mark.gpu


def call_static(L, dt, B, H, Dh, Lmax, q, k, v, kc, vc, out, scale, t, status=None):
    err = C.create_string_buffer(256)
    rc = L.ffa_attention_static_scratch(CODE[dt], B, H, Dh, Lmax, _ptr(q), _ptr(k), _ptr(v), _ptr(kc), _ptr(vc),
                                        _ptr(out), float(scale), int(t), _ptr(status), _stream(), err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("dt,B,H,Dh,Lp", [(torch.float16, 2, 4, 64, 300), (torch.bfloat16, 4, 8, 128, 1000),
                                          (torch.float32, 1, 32, 64, 872), (torch.float16, 1, 2, 80, 37)])
def test_static_scratch_matches_workspace_entry_point(dt, B, H, Dh, Lp):
    L = capi.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    steps = 2
    Lmax = Lp + steps
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    eng = CAbiEngine(K, V, Lmax)                 # regular entry point, caller-allocated workspace
    orc = O.DecodeOracle(K, V, Lmax, compute_dtype=torch.float64)   # and the checker, evaluated in float64
    kc2, vc2 = eng.k_cache.clone(), eng.v_cache.clone()   # same prompt rows for the static-scratch calls
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    scale = 1 / math.sqrt(Dh)
    for i in range(steps):                       # two calls in a row share the static array
        t = Lp + i
        q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt).to(dev) for _ in range(3))
        want = eng.attention(q, k, v, scale, t)
        got = torch.empty(B, H, Dh, dtype=dt, device=dev)
        rc, msg = call_static(L, dt, B, H, Dh, Lmax, q, k, v, kc2, vc2, got, scale, t, status)
        assert rc == 0, msg
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= TOL[dt], (dt, i, err)
        ref = orc.step(q.cpu(), k.cpu(), v.cpu(), scale, t)
        assert_close_ulp(got.cpu(), ref, dt, f"static scratch vs oracle, step {i}")
        assert torch.equal(kc2[:, :, t], k[:, :, 0]) and torch.equal(vc2[:, :, t], v[:, :, 0])
    assert torch.equal(kc2[:, :, :Lmax], eng.k_cache[:, :, :Lmax])
    assert int(status.item()) == 0 and eng.status() == 0


def test_static_scratch_status_word_survives_calls_until_it_is_read():
    """A caller that passes no device_status of its own reads the engine's error bits with
    ffa_static_scratch_status: the word lives in the static array, no decode call clears it,
    reading it does."""
    L = capi.lib()
    dev = torch.device("cuda:0")
    st = C.c_int(-1)
    L.ffa_static_scratch_status(_stream(), C.byref(st))          # whatever earlier tests left: read and clear
    assert L.ffa_static_scratch_status(_stream(), C.byref(st)) == 0 and st.value == 0
    # a bounded wait that runs out (50 ms, on a barrier nothing completes) records the time-out bit ...
    assert L.ffa_static_scratch_selftest_wait_timeout(50, _stream()) == 0
    # ... a clean decode step with device_status == NULL afterwards does not wipe it ...
    dt, B, H, Dh, Lp = torch.float16, 2, 4, 64, 100
    g = torch.Generator().manual_seed(6)
    K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
    eng = CAbiEngine(K, V, Lp + 1)
    q, k, v = (torch.randn(B, H, 1, Dh, generator=g).to(dt).to(dev) for _ in range(3))
    got = torch.empty(B, H, Dh, dtype=dt, device=dev)
    rc, msg = call_static(L, dt, B, H, Dh, Lp + 1, q, k, v, eng.k_cache, eng.v_cache, got, 0.125, Lp, None)
    assert rc == 0, msg
    ref = O.attention_reference(q.cpu().view(B * H, 1, Dh), torch.cat([K, k.cpu()], 2).view(B * H, Lp + 1, Dh),
                                torch.cat([V, v.cpu()], 2).view(B * H, Lp + 1, Dh), 0.125, torch.float64)
    assert_close_ulp(got.cpu().view(B * H, Dh), ref.view(B * H, Dh), dt, "step with NULL device_status")
    # ... the getter reports it (FFA_ERR_DEVICE, bit 1 = time-out) and clears it
    assert L.ffa_static_scratch_status(_stream(), C.byref(st)) == -7 and st.value == 1
    assert L.ffa_static_scratch_status(_stream(), C.byref(st)) == 0 and st.value == 0


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    L = capi.lib()
    dev = torch.device("cuda:0")
    x = torch.zeros(64, dtype=torch.float16, device=dev)
    # batch*heads = 8192 at head_dim 256 needs > 4 MiB of scratch: refused before anything is launched
    rc, msg = call_static(L, torch.float16, 64, 128, 256, 16, x, x, x, x, x, x, 0.0625, 3)
    assert rc == -3 and "static scratch" in msg and "4194304" in msg
    rc, msg = call_static(L, torch.float16, 1, 1, 96, 16, x, x, x, x, x, x, 0.1, 3)
    assert rc == -2 and "head_dim" in msg
    rc, msg = call_static(L, torch.float16, 1, 1, 64, 16, x, x, x, x, x, x, 0.1, 16)
    assert rc == -3
