"""A decode step recorded once in a CUDA graph and replayed for every token.

The per-call host work of `FastForwardAttn.attention` (argument checks, planning, launch)
is a few microseconds -- more than the kernel itself on small configurations.  The row
index can live in device memory (`attention_per_sample`), which makes the launch parameters
of a step independent of the token position, so the step can be captured once:

    step = GraphedStep(ffa, softmax_scale, first_row=prompt_len)
    for token in range(n):
        out = step(q, k, v)          # [B, H, Dh]; a view of a static buffer, valid until the next call

The graph holds: the attention launch on the engine's own caches and the increment of the
row counter.  q, k and v are copied into static buffers before every replay.

The engine lays its work out for an upper bound on the row index that the host states at
launch time.  A graph therefore covers a bucket of rows (bound 127, 255, 511, ... up to the
cache length) and is recorded again, lazily, when the generation enters the next bucket -- a
dozen recordings over a whole generation, each a few hundred microseconds -- so that a mostly
empty cache does not leave most CTAs without rows.
"""
from __future__ import annotations

import torch


def row_bucket(row: int, max_len: int) -> int:
    """Upper bound of the bucket of rows that `row` falls in: 2^k - 1 >= max(row, 127), capped at max_len - 1."""
    bound = 127
    while bound < row:
        bound = 2 * bound + 1
    return min(bound, max_len - 1)


class GraphedStep:
    def __init__(self, ffa, softmax_scale: float, first_row: int, prob_thresh: float = 0.0):
        kc, _ = ffa.get_cache()
        B, H, Lmax, Dh = kc.shape
        if not 0 <= first_row < Lmax:
            raise ValueError(f"first_row {first_row} outside [0, {Lmax})")
        self.ffa, self.max_len = ffa, Lmax
        dev, dt = kc.device, kc.dtype
        self.q = torch.zeros(B, H, 1, Dh, dtype=dt, device=dev)
        self.k = torch.zeros_like(self.q)
        self.v = torch.zeros_like(self.q)
        self.out = torch.zeros(B, H, Dh, dtype=dt, device=dev)
        self.rows = torch.full((B,), first_row, dtype=torch.int32, device=dev)
        self.next_row = first_row
        self.scale, self.p = softmax_scale, prob_thresh
        # warm-up on a side stream (lazy initialisation must not happen inside the capture);
        # it writes row `first_row` with zeros, which the first real step overwrites
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            ffa.attention_per_sample(self.q, self.k, self.v, softmax_scale, self.rows, prob_thresh, out=self.out,
                                     max_row=row_bucket(first_row, Lmax))
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graphs = {}
        self._graph_for(first_row)

    def _graph_for(self, row: int) -> torch.cuda.CUDAGraph:
        bound = row_bucket(row, self.max_len)
        graph = self.graphs.get(bound)
        if graph is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.ffa.attention_per_sample(self.q, self.k, self.v, self.scale, self.rows, self.p, out=self.out, max_row=bound)
                self.rows.add_(1)
            self.graphs[bound] = graph
        return graph

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if self.next_row >= self.max_len:
            raise RuntimeError(f"the cache is full ({self.max_len} rows)")
        graph = self._graph_for(self.next_row)
        self.q.copy_(q.view_as(self.q), non_blocking=True)
        self.k.copy_(k.view_as(self.k), non_blocking=True)
        self.v.copy_(v.view_as(self.v), non_blocking=True)
        graph.replay()
        self.next_row += 1
        return self.out


class GraphedHostStep:
    """A host-driven decode step -- q, k, v arrive in pinned host memory, the result is wanted in
    pinned host memory -- with two host-issued operations per token instead of five:

        step = GraphedHostStep(ffa, softmax_scale, first_row=prompt_len)        # or sharded.graphed_step(...)
        for token in range(n):
            out_host = step(qkv_host)        # qkv_host: pinned [3, B, H, 1, Dh]
            torch.cuda.current_stream().synchronize()    # out_host is valid from here until the next call

    One asynchronous upload of q/k/v into a static device buffer, then one replay of a graph that
    holds the attention launch (row index in device memory; when the heads are sharded -- `gather` =
    the ShardedFastForwardAttn, after enable_peer_gather() -- its epilogue pushes the output rows to
    the peers and a wait-and-collect kernel follows), the increment of the row index, and the download of the result into
    `out_host` ([B, H, Dh], or [B, world*H, Dh] when gathered).  Graphs are recorded per bucket
    of rows, like GraphedStep.
    """

    def __init__(self, ffa, softmax_scale: float, first_row: int, prob_thresh: float = 0.0, gather=None):
        kc, _ = ffa.get_cache()
        B, H, Lmax, Dh = kc.shape
        if not 0 <= first_row < Lmax:
            raise ValueError(f"first_row {first_row} outside [0, {Lmax})")
        self.ffa, self.max_len, self.scale, self.p = ffa, Lmax, softmax_scale, prob_thresh
        self.gather = gather if gather is not None and getattr(gather, "world", 1) > 1 else None
        if self.gather is not None and not self.gather.peer_gather_enabled:
            raise ValueError("a graphed gather needs the peer-memory all-gather: call enable_peer_gather() first")
        dev, dt = kc.device, kc.dtype
        world = self.gather.world if self.gather is not None else 1
        self.stage = torch.zeros(3, B, H, 1, Dh, dtype=dt, device=dev)
        self.local = torch.zeros(B, H, Dh, dtype=dt, device=dev)
        self.full = torch.zeros(B, world * H, Dh, dtype=dt, device=dev) if world > 1 else self.local
        self.out_host = torch.zeros(B, world * H, Dh, dtype=dt).pin_memory()
        self.rows = torch.full((B,), first_row, dtype=torch.int32, device=dev)
        self.next_row = first_row
        self.graphs = {}
        # lazy initialisation (kernel attributes, occupancy answers) outside any capture; writes zeros
        # to row `first_row`, which the first real step overwrites.  No gather here: it is collective.
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            ffa.attention_per_sample(self.stage[0], self.stage[1], self.stage[2], softmax_scale, self.rows, prob_thresh,
                                     out=self.local, max_row=row_bucket(first_row, Lmax))
        torch.cuda.current_stream(dev).wait_stream(side)
        self._graph_for(first_row)

    def _graph_for(self, row: int) -> torch.cuda.CUDAGraph:
        bound = row_bucket(row, self.max_len)
        graph = self.graphs.get(bound)
        if graph is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.ffa.attention_per_sample(self.stage[0], self.stage[1], self.stage[2], self.scale, self.rows, self.p,
                                              out=self.local, max_row=bound,
                                              gather_into=self.full if self.gather is not None else None)
                self.rows.add_(1)
                self.out_host.copy_(self.full, non_blocking=True)
            self.graphs[bound] = graph
        return graph

    def reset_row(self, row: int) -> None:
        """The next step appends at `row` (a new generation over the same caches)."""
        if not 0 <= row < self.max_len:
            raise ValueError(f"row {row} outside [0, {self.max_len})")
        self.rows.fill_(row)
        self.next_row = row

    def __call__(self, qkv_host: torch.Tensor) -> torch.Tensor:
        if self.next_row >= self.max_len:
            raise RuntimeError(f"the cache is full ({self.max_len} rows)")
        graph = self._graph_for(self.next_row)
        self.stage.copy_(qkv_host.view_as(self.stage), non_blocking=True)
        graph.replay()
        self.next_row += 1
        return self.out_host


class GraphedLayers:
    """Every layer's attention for one token -- and whatever the caller computes between the
    layers -- recorded in ONE CUDA graph.

    A decoder runs its layers one after another, each with its own KV cache, and the launch
    and argument-checking cost of L separate calls is what bounds short-sequence decoding
    (the reference's HF forks make one `attention` call per layer per token,
    modeling_opt.py:201-226).  Here the caller hands over one engine per layer and a `body`:

        def body(x, attend):                 # x: the static input tensor of a token
            for i, layer in enumerate(layers):
                q, k, v = layer.project(x)   # any torch ops
                x = x + layer.out_proj(attend(i, q, k, v))    # attend -> [B, H, Dh]
            return x

        step = GraphedLayers(engines, softmax_scale, first_row=prompt_len, body=body, example_input=x0)
        for token in range(n):
            y = step(x)                      # a view of a static buffer, valid until the next call

    `attend(i, q, k, v)` runs engine i with the row index read from device memory; the graph
    ends with one increment of that index, shared by all layers.  `body` is traced once for a
    warm-up (so that libraries it calls create their handles outside the capture) and once per
    bucket of rows for a capture (see the module text); it must be free of host
    synchronisation and of data-dependent control flow, and must return the same kind of
    result every time.  The warm-up writes row `first_row` of every layer's cache, which the
    first real step overwrites.
    """

    def __init__(self, engines, softmax_scale: float, first_row: int, body, example_input: torch.Tensor,
                 prob_thresh: float = 0.0):
        if not engines:
            raise ValueError("need at least one engine")
        shapes = {tuple(e.get_cache()[0].shape) for e in engines}
        if len(shapes) != 1:
            raise ValueError("all layers must share one cache shape")
        kc = engines[0].get_cache()[0]
        B, H, Lmax, Dh = kc.shape
        if not 0 <= first_row < Lmax:
            raise ValueError(f"first_row {first_row} outside [0, {Lmax})")
        dev = kc.device
        self.engines, self.max_len, self.next_row = list(engines), Lmax, first_row
        self.x = example_input.detach().clone().to(dev)
        self.rows = torch.full((B,), first_row, dtype=torch.int32, device=dev)
        self.outs = [torch.zeros(B, H, Dh, dtype=kc.dtype, device=dev) for _ in engines]
        self.body, self.scale, self.p = body, softmax_scale, prob_thresh

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            body(self.x, self._attend(row_bucket(first_row, Lmax)))
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graphs = {}
        self._graph_for(first_row)

    def _attend(self, bound: int):
        def attend(i: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
            return self.engines[i].attention_per_sample(q, k, v, self.scale, self.rows, self.p, out=self.outs[i], max_row=bound)

        return attend

    def _graph_for(self, row: int):
        bound = row_bucket(row, self.max_len)
        entry = self.graphs.get(bound)
        if entry is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"), torch.no_grad():
                y = self.body(self.x, self._attend(bound))
                self.rows.add_(1)
            entry = self.graphs[bound] = (graph, y)
        return entry

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.next_row >= self.max_len:
            raise RuntimeError(f"the caches are full ({self.max_len} rows)")
        graph, y = self._graph_for(self.next_row)
        self.x.copy_(x, non_blocking=True)
        graph.replay()
        self.next_row += 1
        return y
