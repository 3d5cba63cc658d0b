"""What a pruned step costs against the share of rows its threshold keeps.

The reference's pruning skips V loads only (attention.cu:1184-1191), so a threshold that prunes
nothing costs it nothing extra.  Here a pruned step needs the softmax statistics before the first
V row; fetching survivors row by row pays when most rows are pruned and costs when they are not,
which is why a slice that keeps 45 % or more of its rows streams its V tiles instead.  This test
times random keys with queries scaled so that p = 1e-3 keeps everything, about half, or a few
per cent of the rows (CUDA-graph replay over rotating replicas, every launch from HBM), prints
the table and asserts the two ends: pruning must pay when it prunes, and must not cost more than
a third on top of the exact step when it does not.
"""
import pytest
import torch

from tests.helpers import report

pytestmark = pytest.mark.gpu

SHAPES = [("fp16 B10 H32 Dh64, 1256 tokens", torch.float16, 10, 32, 64, 1256, 6),
          ("bf16 B32 H32 Dh128, 2048 tokens", torch.bfloat16, 32, 32, 128, 2048, 2)]


def _replay_us(step, nrep, launches=32):
    for i in range(nrep):
        step(i)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            step(i)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / launches * 1e3


@pytest.mark.parametrize("name,dt,B,H,Dh,L,nrep", SHAPES, ids=[s[0].split(",")[0].replace(" ", "-") for s in SHAPES])
def test_pruned_step_against_kept_share(name, dt, B, H, Dh, L, nrep):
    from fastforwardattention_b200 import FastForwardAttn

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(3)
    engines = []
    for _ in range(nrep):
        K = torch.randn(B, H, L - 1, Dh, generator=g, device=dev, dtype=dt)
        V = torch.randn(B, H, L - 1, Dh, generator=g, device=dev, dtype=dt)
        engines.append(FastForwardAttn(K, V, L, False))
        del K, V
    k = torch.randn(B, H, 1, Dh, generator=g, device=dev).to(dt)
    out = torch.empty(B, H, Dh, dtype=dt, device=dev)
    t, scale, p = L - 1, Dh ** -0.5, 1e-3
    rows = []
    for qscale in (1.0, 2.0, 4.0):
        q = (qscale * torch.randn(B, H, 1, Dh, generator=torch.Generator(device=dev).manual_seed(11), device=dev)).to(dt)

        def exact(i):
            engines[i % nrep].attention(q, k, k, scale, t, 0.0, out=out)

        def pruned(i):
            engines[i % nrep].attention(q, k, k, scale, t, p, out=out)

        us_exact, us_pruned = _replay_us(exact, nrep), _replay_us(pruned, nrep)
        e = engines[0]
        e.record_kept_mask(True)
        e.attention(q, k, k, scale, t, p, out=out)
        m = e.get_kept_mask()
        e.record_kept_mask(False)
        kept = sum(int(((m.view(-1) >> i) & 1).sum()) for i in range(32)) / (B * H * L)
        rows.append((kept, us_exact, us_pruned))
    report(f"pruned step against the share of rows kept, {name} (us per step):")
    for kept, us_exact, us_pruned in rows:
        report(f"  keeps {100 * kept:5.1f} %   exact {us_exact:7.1f}   pruned {us_pruned:7.1f}   ratio {us_pruned / us_exact:4.2f}")
    assert max(e.device_status() for e in engines) == 0
    dense, sparse = rows[0], rows[-1]
    assert dense[0] > 0.95 and sparse[0] < 0.15, rows
    assert sparse[2] < sparse[1], ("pruning must pay when it prunes", rows)
    assert dense[2] < 1.33 * dense[1], ("a threshold that prunes nothing must not cost more than a third", rows)
