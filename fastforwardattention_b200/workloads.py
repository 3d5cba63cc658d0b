"""Seeded synthetic decode-attention workloads.

The reference measures on OPT-1.3B / GPT-J generation over a summarisation dataset
(summarize.py:29-145); model weights and the dataset are not available offline, so tensors
of the same shapes and an N(0,1) value distribution stand in for the projected q/k/v.  The
generators are deterministic in (name, seed) and produce CPU tensors; callers move them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Iterator, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    dtype: torch.dtype
    B: int
    H: int
    Dh: int
    prompt: int
    steps: int
    p: float = 0.0
    seed: int = 1234
    peaked: bool = False  # pruning workload: 5 % of positions carry q-aligned keys

    @property
    def max_len(self) -> int:
        return self.prompt + self.steps

    @property
    def scale(self) -> float:
        return 1.0 / math.sqrt(self.Dh)

    def shard(self, rank: int, world: int) -> "Workload":
        """The head shard rank `rank` of `world` owns: heads [rank*H/world, (rank+1)*H/world)."""
        assert self.H % world == 0, "head count must divide by the number of GPUs"
        return replace(self, name=f"{self.name}/r{rank}of{world}", H=self.H // world,
                       seed=self.seed * 1000 + rank)


def long_sweep(x: int) -> Workload:
    """bf16, batch 32, 32 heads, head_dim 128, final length x (prompt x-128, 128 steps)."""
    return Workload(f"long-bf16-b32-h32-d128-L{x}", torch.bfloat16, 32, 32, 128, x - 128, 128, seed=1239)


CONFIGS = {
    "opt13b-fp32-b1": Workload("opt13b-fp32-b1", torch.float32, 1, 32, 64, 872, 128, seed=1235),
    "opt13b-fp16-b10": Workload("opt13b-fp16-b10", torch.float16, 10, 32, 64, 1000, 256, seed=1236),
    "gptj-fp16-b8": Workload("gptj-fp16-b8", torch.float16, 8, 16, 256, 1920, 128, seed=1237),
    "prune-fp16-b10-p1e-4": Workload("prune-fp16-b10-p1e-4", torch.float16, 10, 32, 64, 1000, 256, p=1e-4,
                                     seed=1238, peaked=True),
    "prune-fp16-b10-p1e-3": Workload("prune-fp16-b10-p1e-3", torch.float16, 10, 32, 64, 1000, 256, p=1e-3,
                                     seed=1238, peaked=True),
    **{f"long-{x}": long_sweep(x) for x in (512, 2048, 8192, 32768)},
    # the long-sequence shapes with peaked keys and a threshold: what pruning is for at lengths the reference cannot reach
    **{f"prune-long-{x}": replace(long_sweep(x), name=f"prune-long-bf16-b32-h32-d128-L{x}", p=1e-3, seed=1240, peaked=True)
       for x in (8192, 32768)},
}


def prompt_kv(w: Workload, device="cpu", chunk_bh: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Prompt K and V, [B, H, prompt, Dh] in w.dtype.  Generated per (batch, head) chunk in
    fp32 then cast, so that the 32 K-token case never needs an fp32 copy of the whole cache."""
    g = torch.Generator(device="cpu").manual_seed(w.seed)
    N = w.B * w.H
    K = torch.empty(N, w.prompt, w.Dh, dtype=w.dtype, device=device)
    V = torch.empty(N, w.prompt, w.Dh, dtype=w.dtype, device=device)
    for i in range(0, N, chunk_bh):
        n = min(chunk_bh, N - i)
        k = torch.randn(n, w.prompt, w.Dh, generator=g)
        v = torch.randn(n, w.prompt, w.Dh, generator=g)
        if w.peaked:
            q0 = _base_query(w)[i:i + n]
            peak = torch.rand(n, w.prompt, generator=g) < 0.05
            k = torch.where(peak[..., None], 4.0 * q0[:, None, :], 0.5 * k)
        K[i:i + n] = k.to(w.dtype)
        V[i:i + n] = v.to(w.dtype)
    return K.view(w.B, w.H, w.prompt, w.Dh), V.view(w.B, w.H, w.prompt, w.Dh)


def _base_query(w: Workload) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(w.seed + 7919)
    return torch.randn(w.B * w.H, w.Dh, generator=g)


def step_qkv(w: Workload) -> Iterator[Tuple[int, torch.Tensor, torch.Tensor, torch.Tensor]]:
    """Yields (t, q, k, v) for t = prompt .. prompt+steps-1; q, k, v are [B, H, 1, Dh]."""
    g = torch.Generator(device="cpu").manual_seed(w.seed + 104729)
    N = w.B * w.H
    q0 = _base_query(w) if w.peaked else None
    for i in range(w.steps):
        q = torch.randn(N, w.Dh, generator=g)
        k = torch.randn(N, w.Dh, generator=g)
        v = torch.randn(N, w.Dh, generator=g)
        if w.peaked:
            q = q0 + 0.25 * q
            peak = torch.rand(N, generator=g) < 0.05
            k = torch.where(peak[:, None], 4.0 * q0, 0.5 * k)
        shape = (w.B, w.H, 1, w.Dh)
        yield w.prompt + i, q.to(w.dtype).view(shape), k.to(w.dtype).view(shape), v.to(w.dtype).view(shape)


def device_prompt_kv(w: Workload, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Prompt K and V generated directly in device memory (benchmark sizes: 8.6 GB per tensor
    at 32 K tokens would take minutes through the host generator).  Values are N(0,1); the
    pruning workload puts 4*q0 on a seeded 5 % of the positions and N(0, 0.5) elsewhere."""
    g = torch.Generator(device=device).manual_seed(w.seed)
    shape = (w.B, w.H, w.prompt, w.Dh)
    K = torch.empty(shape, dtype=w.dtype, device=device)
    V = torch.empty(shape, dtype=w.dtype, device=device)
    q0 = _base_query(w).to(device).view(w.B, w.H, 1, w.Dh) if w.peaked else None
    for b in range(w.B):
        K[b].normal_(generator=g)
        V[b].normal_(generator=g)
        if w.peaked:
            peak = torch.rand(w.H, w.prompt, 1, generator=g, device=device) < 0.05
            K[b] = torch.where(peak, (4.0 * q0[b]).to(w.dtype), (0.5 * K[b].float()).to(w.dtype))
    return K, V


def device_step_qkv(w: Workload, steps: int, device) -> torch.Tensor:
    """[steps, 3, B, H, 1, Dh] of q, k, v for `steps` decode steps, generated on the device
    with the same distributions as step_qkv (not the same values)."""
    g = torch.Generator(device=device).manual_seed(w.seed + 1)
    x = torch.randn(steps, 3, w.B, w.H, 1, w.Dh, generator=g, device=device, dtype=torch.float32)
    if w.peaked:
        q0 = _base_query(w).to(device).view(1, w.B, w.H, 1, w.Dh)
        x[:, 0] = q0 + 0.25 * x[:, 0]
        peak = torch.rand(steps, w.B, w.H, 1, 1, generator=g, device=device) < 0.05
        x[:, 1] = torch.where(peak, 4.0 * q0, 0.5 * x[:, 1])
    return x.to(w.dtype)
