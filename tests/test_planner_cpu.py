"""The launch planner's rules, checked without a GPU through an offline plan that is told the
B200's multiprocessor count and shared-memory limits."""
import ctypes as C
import itertools

import pytest

from fastforwardattention_b200 import capi

SMS, SMEM_CTA, SMEM_SM = 148, 232448, 233472
ES = {capi.F32: 4, capi.F16: 2, capi.BF16: 2}


def offline(dtype, B, H, Dh, Lmax, use_default=0, sms=SMS):
    L = capi.lib()
    p = C.c_void_p()
    capi.check(L.ffa_plan_create_offline(dtype, B, H, Dh, Lmax, use_default, sms, SMEM_CTA, SMEM_SM, C.byref(p)))
    return L, p


def launch(L, p, t):
    l = capi.Launch()
    capi.check(L.ffa_plan_get_launch(p, t, C.byref(l)))
    return l


@pytest.mark.parametrize("dtype,Dh", list(itertools.product([capi.F32, capi.F16, capi.BF16], [64, 80, 128, 256])))
def test_every_shape_fits_and_covers_the_work(dtype, Dh):
    for B, H, Lmax in [(1, 1, 1), (1, 32, 1000), (10, 32, 1256), (8, 16, 2048), (32, 32, 32768), (64, 64, 300), (1, 4, 200000)]:
        L, p = offline(dtype, B, H, Dh, Lmax)
        for t in sorted({0, 1, 7, 8, 9, Lmax // 2, Lmax - 1}):
            if t >= Lmax:
                continue
            l = launch(L, p, t)
            assert l.tile_rows % 8 == 0 and l.tile_rows >= 8
            assert 2 <= l.stages <= 16 and 1 <= l.consumer_warps <= 8
            assert l.smem_bytes <= SMEM_CTA and l.ctas_per_sm * (l.smem_bytes + 1024) <= SMEM_SM
            units = B * H * (t // l.tile_rows + 1)
            assert 1 <= l.grid <= min(units, SMS * 8)            # no CTA without a unit
            assert l.grid <= SMS * l.ctas_per_sm
            upb = t // l.tile_rows + 1
            assert 1 <= l.parts_per_bh <= upb and l.grid <= B * H * l.parts_per_bh   # every CTA owns whole parts
            # the ring really holds stages x (K tile + V tile)
            assert l.smem_bytes >= l.stages * 2 * l.tile_rows * Dh * ES[dtype]
        L.ffa_plan_destroy(p)


def test_benchmark_configurations_get_the_measured_shapes():
    # config 5 at 32 K tokens: 16 KB tiles, 2-stage ring, 4 compute warps, 2 CTAs per SM
    L, p = offline(capi.BF16, 32, 32, 128, 32768)
    l = launch(L, p, 32767)
    assert (l.tile_rows, l.stages, l.consumer_warps, l.ctas_per_sm, l.grid) == (64, 2, 4, 2, 296)
    assert l.parts_per_bh == 32767 // 64 + 1           # large problem: even cut of the unit list
    # config 1 (16 MB per step, 32 pairs): two CTAs per SM, 8 CTAs per (batch, head) = one thread-block cluster, boundaries aligned
    L, p = offline(capi.F32, 1, 32, 64, 1000)
    l = launch(L, p, 999)
    assert (l.ctas_per_sm, l.grid, l.parts_per_bh) == (2, 256, 8)
    # config 2: a third resident CTA per SM makes room for one CTA per (batch, head)
    L, p = offline(capi.F16, 10, 32, 64, 1256)
    l = launch(L, p, 1255)
    assert (l.ctas_per_sm, l.grid, l.parts_per_bh) == (3, 320, 1)
    # config 3 (GPT-J rows of 512 bytes, 269 MB): 8 compute warps
    L, p = offline(capi.F16, 8, 16, 256, 2048)
    assert launch(L, p, 2047).consumer_warps == 8
    # the analytic rule ignores the refinements
    L, p = offline(capi.F32, 1, 32, 64, 1000, use_default=1)
    assert launch(L, p, 999).ctas_per_sm == 2
    # 16 pairs on 148 SMs: 9 CTAs per pair would fit, 8 are taken so that a pair is one thread-block cluster;
    # without the cluster merge the ninth is used
    L, p = offline(capi.F16, 1, 16, 256, 2048)
    l = launch(L, p, 2047)
    assert (l.grid, l.parts_per_bh) == (128, 8)
    capi.check(L.ffa_plan_set_cluster_merge(p, 0))
    l = launch(L, p, 2047)
    assert (l.grid, l.parts_per_bh) == (144, 9)
    # 8 pairs: 18 CTAs per pair would fit; 16 are taken = two whole clusters of 8 per pair, whose
    # leaders merge through global memory
    L, p = offline(capi.BF16, 2, 4, 128, 8192)
    l = launch(L, p, 8191)
    assert (l.grid, l.parts_per_bh) == (128, 16)
    # 4 pairs at 32 K tokens: at most 12 clusters of 8 per pair
    L, p = offline(capi.BF16, 1, 4, 128, 32768)
    l = launch(L, p, 32767)
    assert (l.grid, l.parts_per_bh) == (384, 96)


def test_forced_shape_is_respected_and_clamped():
    L, p = offline(capi.F16, 2, 4, 64, 500)
    f = capi.Launch(16, 3, 2, 4, 5, 0, 0)
    capi.check(L.ffa_plan_set_launch(p, C.byref(f)))
    l = launch(L, p, 400)
    assert (l.tile_rows, l.stages, l.consumer_warps, l.ctas_per_sm, l.grid) == (16, 3, 2, 4, 5)
    f = capi.Launch(100000, 99, 99, 99, 0, 0, 0)        # absurd: clamped until it fits
    capi.check(L.ffa_plan_set_launch(p, C.byref(f)))
    l = launch(L, p, 400)
    assert l.smem_bytes <= SMEM_CTA and l.consumer_warps == 8 and l.stages >= 2
    capi.check(L.ffa_plan_set_launch(p, None))
    assert launch(L, p, 400).consumer_warps == 4


def test_offline_plan_cannot_launch_and_range_checks():
    L, p = offline(capi.F16, 2, 4, 64, 500)
    l = capi.Launch()
    assert L.ffa_plan_get_launch(p, 500, C.byref(l)) == -3
    x = C.c_void_p(256)
    assert L.ffa_attention(p, x, x, x, x, x, x, 1.0, 0, None, 1, 0.0, None, None) == -4
    assert b"offline" in L.ffa_last_error()
    q = C.c_void_p()
    assert L.ffa_plan_create_offline(capi.F16, 2, 4, 64, 500, 0, 0, SMEM_CTA, SMEM_SM, C.byref(q)) == -3


def prune_launch(L, p, t):
    v = [C.c_int() for _ in range(5)]
    capi.check(L.ffa_plan_get_prune_launch(p, t, *[C.byref(x) for x in v]))
    return tuple(x.value for x in v)     # cluster, chunk_rows, tile_rows, grid, smem


def test_fused_pruning_launch_rules():
    # config 4: clusters of 2, everything resident in one wave
    L, p = offline(capi.F16, 10, 32, 64, 1256)
    c, chunk, r, grid, smem = prune_launch(L, p, 1255)
    assert (c, chunk, grid) == (2, 640, 640) and smem <= 48 * 1024
    assert grid <= SMS * min(7, SMEM_SM // (smem + 1024))
    # few pairs: slice up to 8 ways but never below 128 rows
    L, p = offline(capi.F32, 1, 32, 64, 1000)
    c, chunk, r, grid, smem = prune_launch(L, p, 999)
    assert c == 8 and chunk == 128
    # long sequences: slices sized so several CTAs share an SM
    L, p = offline(capi.BF16, 32, 32, 128, 32768)
    c, chunk, r, grid, smem = prune_launch(L, p, 32767)
    assert c >= 2 and chunk * c >= 32768 and chunk % 32 == 0 and smem <= SMEM_CTA
    assert SMEM_SM // (smem + 1024) >= 2
    # a sequence no 8 slices can hold in shared memory falls back to the streaming kernel
    L, p = offline(capi.F32, 1, 1, 64, 2000000)
    assert prune_launch(L, p, 1999999) == (0, 0, 0, 0, 0)
    for t in (0, 1, 31, 32, 33, 500):
        L, p = offline(capi.F16, 3, 5, 80, 501)
        c, chunk, r, grid, smem = prune_launch(L, p, t)
        assert c >= 1 and chunk % 32 == 0 and chunk * c >= t + 1 and r % 8 == 0 and grid == 15 * c


def prune_path(L, p, t, thresh, with_scores=1):
    v = C.c_int()
    capi.check(L.ffa_plan_get_prune_path(p, t, thresh, with_scores, C.byref(v)))
    return v.value


def test_which_pruning_kernel_a_step_takes():
    # config 4 (51 MB of K): the cluster kernel
    L, p = offline(capi.F16, 10, 32, 64, 1256)
    assert prune_path(L, p, 1255, 1e-3) == 1
    # bf16 B32 H32 Dh128: 2 K tokens stream 537 MB of K (cluster kernel), 8 K tokens 2.1 GB (streaming kernel)
    L, p = offline(capi.BF16, 32, 32, 128, 32768)
    assert prune_path(L, p, 2047, 1e-3) == 1
    assert prune_path(L, p, 8191, 1e-3) == 2
    assert prune_path(L, p, 8191, 1e-3, with_scores=0) == 1      # no score scratch bound: the cluster kernel whenever it fits
    assert prune_path(L, p, 32767, 0.0) == 1                     # torch rounding, every row kept: always the cluster kernel
    capi.check(L.ffa_plan_set_prune_path(p, 2))
    assert prune_path(L, p, 100, 1e-3) == 2
    capi.check(L.ffa_plan_set_prune_path(p, 1))
    assert prune_path(L, p, 32767, 1e-3) == 1
    # a sequence no 8 slices can hold in shared memory: the streaming kernel, or nothing without the scratch
    L, p = offline(capi.F32, 1, 1, 64, 2000000)
    assert prune_path(L, p, 1999999, 1e-3) == 2
    assert prune_path(L, p, 1999999, 1e-3, with_scores=0) == 0
