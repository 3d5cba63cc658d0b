"""Head-sharded decode attention across the GPUs of one node.

Every (batch, head) pair is an independent problem (the reference's grid is one CTA per
pair, attention.cu:1303), so rank r of N owns heads [r*H/N, (r+1)*H/N) for the whole
generation: its slice of the prompt K/V, its KV-cache shard, its slice of every q/k/v.  No
cache row ever crosses NVLink.  The only collective is one all-gather of the [B, H/N, Dh]
outputs, issued when the caller asks for the full [B, H, Dh] tensor: through the process
group (NCCL), or -- after enable_peer_gather() -- by the engine's own kernels: the attention
kernel stores every output row, as it produces it, straight into the peers' memory, and a
short second kernel waits for the peers' rows and puts them in place (no permutation).

One process per GPU (torchrun); the process group decides the backend (NCCL on GPUs).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_range(num_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """Heads [lo, hi) owned by `rank`."""
    if num_heads % world != 0:
        raise ValueError(f"{num_heads} heads do not divide over {world} ranks")
    per = num_heads // world
    return rank * per, (rank + 1) * per


def shard_heads(x: torch.Tensor, rank: int, world: int, num_heads: int) -> torch.Tensor:
    """Slice this rank's heads out of a full tensor.  Accepts [B, H, ...] (example.py:31-33) or
    the HF forks' [B, 1, H*Dh] (modeling_opt.py:193-203)."""
    lo, hi = head_range(num_heads, rank, world)
    if x.dim() >= 3 and x.size(1) == num_heads:
        return x[:, lo:hi].contiguous()
    B = x.size(0)
    return x.reshape(B, num_heads, -1)[:, lo:hi].contiguous()


class ShardedFastForwardAttn:
    """FastForwardAttn over a head shard, plus the optional output all-gather.

    K_local / V_local: this rank's [B, H/N, prompt, Dh] slice.  `engine_factory` builds the
    per-rank engine; it defaults to the CUDA extension and exists so that the host logic can
    be exercised on CPU ranks with a stand-in engine.
    """

    def __init__(self, K_local: torch.Tensor, V_local: torch.Tensor, max_len: int,
                 use_default_kernel_launch: bool = False, group: Optional[dist.ProcessGroup] = None,
                 engine_factory: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if engine_factory is None:
            from . import FastForwardAttn as engine_factory  # raises if the extension is missing
        self.engine = engine_factory(K_local, V_local, max_len, use_default_kernel_launch)
        self.B, self.H_local, _, self.Dh = K_local.shape
        self.H = self.H_local * self.world
        self._gathered = None
        self._peer = False

    def get_cache(self):
        return self.engine.get_cache()

    def attention(self, q_local, k_local, v_local, softmax_scale: float, curr_timestep: int,
                  prob_thresh: float = 0.0, gather: bool = False) -> torch.Tensor:
        """One decode step on this rank's heads; q/k/v hold B*(H/N)*Dh elements.  Returns the
        local [B, H/N, Dh] output, or the full [B, H, Dh] tensor when gather=True."""
        if gather and self._peer:
            # the attention kernel pushes its rows to the peers as it produces them; a short wait-and-collect kernel follows
            return self.engine.attention(q_local, k_local, v_local, softmax_scale, curr_timestep, prob_thresh,
                                         gather_into=self._full(q_local))
        out = self.engine.attention(q_local, k_local, v_local, softmax_scale, curr_timestep, prob_thresh)
        return self.gather(out) if gather else out

    def _full(self, like: torch.Tensor) -> torch.Tensor:
        kc = self.engine.get_cache()[0]   # q may live in pinned host memory; the result goes where the caches are
        return torch.empty(self.B, self.H, self.Dh, dtype=kc.dtype, device=kc.device)

    def enable_peer_gather(self) -> bool:
        """Switch gather() to the engine's peer-memory all-gather.  Collective: every rank of the
        group calls it.  Each rank allocates one small device buffer, the ranks exchange the
        buffers' inter-process handles through the group and map each other's memory.  Returns
        False -- on every rank alike, and gather() keeps using the process group -- when any
        rank could not allocate, export or map a buffer."""
        if self.world == 1 or self._peer:
            return self._peer
        eng, handle = self.engine, None
        try:
            handle = bytes(eng.peer_gather_alloc(self.world))
        except RuntimeError:
            pass
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=self.group)
        ptrs, ok = [], handle is not None and all(h is not None for h in handles)
        if ok:
            try:
                for r, h in enumerate(handles):
                    ptrs.append(eng.peer_gather_ptr() if r == self.rank else eng.peer_mem_open(h))
            except RuntimeError:
                ok = False
        oks = [None] * self.world
        dist.all_gather_object(oks, ok, group=self.group)
        if all(oks):
            eng.peer_gather_attach(self.world, self.rank, ptrs, True)
            self._peer = True
            return True
        for r, p in enumerate(ptrs):
            if r != self.rank:
                eng.peer_mem_close(p)
        dist.barrier(group=self.group)   # nobody still maps another rank's buffer
        if handle is not None:
            eng.peer_gather_free()
        return False

    @property
    def peer_gather_enabled(self) -> bool:
        return self._peer

    def graphed_step(self, softmax_scale: float, first_row: int, prob_thresh: float = 0.0):
        """A whole host-driven step of this rank -- upload of its q/k/v slice, attention, all-gather
        over peer memory, download of the full [B, H, Dh] result -- as one upload plus one CUDA
        graph replay (see GraphedHostStep).  Needs enable_peer_gather(); every rank must then call
        the step the same number of times."""
        from .graphed import GraphedHostStep

        return GraphedHostStep(self.engine, softmax_scale, first_row, prob_thresh, gather=self)

    def close(self) -> None:
        """Collective: releases the peer-gather buffers.  Every rank finishes its queued work and
        meets at a barrier (no store can still be aimed at anyone's buffer), unmaps the peers'
        buffers, meets again (an exported buffer must outlive every mapping of it), and frees
        its own."""
        if not self._peer:
            return
        kc = self.engine.get_cache()[0]
        if kc.is_cuda:
            torch.cuda.synchronize(kc.device)
        dist.barrier(group=self.group)
        self.engine.peer_gather_detach()
        dist.barrier(group=self.group)
        self.engine.peer_gather_free()
        self._peer = False

    def gather(self, out_local: torch.Tensor) -> torch.Tensor:
        """All-gather of the per-rank outputs into [B, H, Dh] (rank-major heads)."""
        if self.world == 1:
            return out_local
        out_local = out_local.contiguous()
        if self._peer:
            return self.engine.peer_gather(out_local)
        if self._gathered is None or self._gathered.dtype != out_local.dtype or self._gathered.device != out_local.device:
            self._gathered = torch.empty(self.world, self.B, self.H_local, self.Dh, dtype=out_local.dtype,
                                         device=out_local.device)
        dist.all_gather_into_tensor(self._gathered.view(-1), out_local.view(-1), group=self.group)
        # [N, B, H/N, Dh] -> [B, N, H/N, Dh] -> [B, H, Dh]
        return self._gathered.permute(1, 0, 2, 3).reshape(self.B, self.H, self.Dh)
