"""Paged KV caches: sequences of different lengths share one pool and take pages as they grow.

The reference allocates `max_len` rows for every sequence at construction
(torch_ffa_api.cpp:65-66); with many concurrent sequences of unknown final length that is
mostly unused memory.  Here a pool of fixed-size pages ([pages, heads, page_rows, head_dim] for
K and for V) is shared; every sequence has a row of the page table and gets a new page only
when its next token crosses a page boundary.  Exact attention and the pruned step
(prob_thresh > 0) both run over the pool.

    pool = PagePool(num_pages=4096, heads=32, head_dim=128, dtype=torch.bfloat16, device="cuda")
    seqs = PagedFastForwardAttn(pool, K, V, max_len=32768, lengths=prompt_lengths)   # K, V: [B, H, Lp, Dh]
    out = seqs.attention(q, k, v, softmax_scale)        # every sequence appends at its own length
    seqs.release()                                      # pages go back to the pool
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


class PagePool:
    """K and V page pools plus a free list.  page_rows must be a multiple of 128."""

    def __init__(self, num_pages: int, heads: int, head_dim: int, dtype: torch.dtype, device, page_rows: int = 256):
        if page_rows % 128 != 0:
            raise ValueError("page_rows must be a multiple of 128")
        self.page_rows, self.heads, self.head_dim = page_rows, heads, head_dim
        self.k = torch.empty(num_pages, heads, page_rows, head_dim, dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        self._free: List[int] = list(range(num_pages - 1, -1, -1))

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise MemoryError("the page pool is exhausted")
        return self._free.pop()

    def release(self, pages: Sequence[int]) -> None:
        self._free.extend(int(p) for p in pages)


class PagedFastForwardAttn:
    """B sequences over a shared PagePool.  K, V: [B, H, Lp, Dh] prompts, right-padded when
    `lengths` (per-sequence prompt lengths) is given."""

    def __init__(self, pool: PagePool, K: torch.Tensor, V: torch.Tensor, max_len: int,
                 lengths: Optional[Sequence[int]] = None, use_default_kernel_launch: bool = False):
        from . import _extension

        B, H, Lp, Dh = K.shape
        if (H, Dh) != (pool.heads, pool.head_dim) or K.dtype != pool.k.dtype:
            raise ValueError("prompt tensors do not match the pool's heads / head_dim / dtype")
        self.pool, self.B = pool, B
        pr = pool.page_rows
        self.max_pages = -(-max_len // pr)
        self.lengths = [Lp] * B if lengths is None else [int(x) for x in lengths]
        if any(not 0 <= n <= Lp for n in self.lengths):
            raise ValueError("lengths must lie in [0, prompt length]")
        dev = pool.k.device
        self.table_host = torch.full((B, self.max_pages), -1, dtype=torch.int32)
        for b, n in enumerate(self.lengths):
            for i in range(-(-n // pr)):
                page = pool.alloc()
                self.table_host[b, i] = page
                rows = min(pr, n - i * pr)
                pool.k[page, :, :rows] = K[b, :, i * pr: i * pr + rows].to(dev)
                pool.v[page, :, :rows] = V[b, :, i * pr: i * pr + rows].to(dev)
        self.table = self.table_host.to(dev)
        self.rows = torch.tensor(self.lengths, dtype=torch.int32, device=dev)
        self.engine = _extension().PagedEngine(pool.k, pool.v, B, self.max_pages, use_default_kernel_launch)

    def _ensure_page(self, b: int, row: int) -> None:
        i = row // self.pool.page_rows
        if i >= self.max_pages:
            raise RuntimeError(f"sequence {b} is full ({self.max_pages * self.pool.page_rows} rows)")
        if self.table_host[b, i] < 0:
            page = self.pool.alloc()
            self.table_host[b, i] = page
            self.table[b, i] = page

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                  prob_thresh: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode step: sequence b appends k, v at row lengths[b] and attends rows 0..lengths[b];
        prob_thresh means what it means in FastForwardAttn.attention."""
        for b, n in enumerate(self.lengths):
            if n % self.pool.page_rows == 0:
                self._ensure_page(b, n)
        res = self.engine.attention_per_sample(q, k, v, self.table, softmax_scale, self.rows, prob_thresh, out=out,
                                               max_row=max(self.lengths))
        self.rows += 1
        self.lengths = [n + 1 for n in self.lengths]
        return res

    @property
    def pages_in_use(self) -> int:
        return int((self.table_host >= 0).sum())

    def release(self) -> None:
        self.pool.release(self.table_host[self.table_host >= 0].tolist())
        self.table_host.fill_(-1)
        self.table.fill_(-1)
