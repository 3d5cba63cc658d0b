"""B200-native decode masked multi-head attention behind the FastForwardAttention interface.

    from fastforwardattention_b200 import FastForwardAttn      # or: from ff_attention import FastForwardAttn
    ffa = FastForwardAttn(K, V, prompt_len + output_len, False)
    out = ffa.attention(q, k, v, softmax_scale, t, 0)

There is no CPU path and no fallback: the class lives in the compiled extension
(`python -m fastforwardattention_b200.build`), and importing it without that extension raises.
"""
from __future__ import annotations

import importlib

__all__ = ["FastForwardAttn", "ShardedFastForwardAttn", "GraphedStep", "GraphedHostStep", "GraphedLayers", "PagePool", "PagedFastForwardAttn", "launch_count"]


def _extension():
    try:
        return importlib.import_module(".ff_attention", __name__)
    except ImportError as e:  # fail loudly: nothing else can compute the attention step
        raise ImportError(
            "fastforwardattention_b200: the compiled extension is missing or does not load "
            f"({e}). Build it with `python -m fastforwardattention_b200.build`."
        ) from e


def __getattr__(name):
    if name == "FastForwardAttn":
        return _extension().FastForwardAttn
    if name == "launch_count":
        return _extension().launch_count
    if name in ("PagePool", "PagedFastForwardAttn"):
        from . import paged

        return getattr(paged, name)
    if name == "GraphedLayers":
        from .graphed import GraphedLayers

        return GraphedLayers
    if name in ("GraphedStep", "GraphedHostStep"):
        from . import graphed

        return getattr(graphed, name)
    if name == "ShardedFastForwardAttn":
        from .sharded import ShardedFastForwardAttn

        return ShardedFastForwardAttn
    raise AttributeError(name)
