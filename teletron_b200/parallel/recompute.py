"""Activation recompute / CPU offload policy for a stack of transformer blocks.

Same policies as the reference mixin (teletron/core/transformer/transformer_block.py:6-98):
``recompute_granularity == "full"`` during training selects
  * ``uniform``: checkpoint consecutive chunks of ``recompute_num_layers`` blocks,
  * ``block``  : checkpoint each of the first ``recompute_num_layers`` blocks, run the rest plainly,
both with non-reentrant ``torch.utils.checkpoint``; ``activation_offload`` additionally keeps
the remaining saved tensors in pinned host memory (``save_on_cpu``).  Here it is a function
over (blocks, hidden, extra args) instead of a forward-swapping mixin.  With 180 GB per GPU
the 1.3B model trains without recompute; the policy exists for the 14B / long-video configs.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import Sequence

import torch
from torch.utils.checkpoint import checkpoint


_DISCARDED_FORWARD = False


def forward_is_discarded() -> bool:
    """True inside the first forward pass of a checkpointed range, whose saved activations are dropped
    (they are produced again by the recompute pass right before the range's backward).  Allocators that
    keep per-layer activations outside autograd (the symmetric slab of the fused Ulysses path) use it to
    recycle their space at once."""
    return _DISCARDED_FORWARD


def _run_range(blocks: Sequence, start: int, end: int, extra):
    def fn(x):
        for i in range(start, end):
            x = blocks[i](x, *extra)
        return x

    return fn


def _checkpointed(blocks: Sequence, start: int, end: int, extra, x):
    inner = _run_range(blocks, start, end, extra)
    calls = [0]

    def fn(x):
        global _DISCARDED_FORWARD
        first = calls[0] == 0
        calls[0] += 1
        prev = _DISCARDED_FORWARD
        _DISCARDED_FORWARD = first
        try:
            return inner(x)
        finally:
            _DISCARDED_FORWARD = prev

    return checkpoint(fn, x, use_reentrant=False)


def run_blocks(blocks: Sequence, x, extra: tuple, cfg, training: bool):
    """Apply ``blocks[i](x, *extra)`` in order under the recompute policy in ``cfg``."""
    n = len(blocks)
    full = training and getattr(cfg, "recompute_granularity", None) == "full" and torch.is_grad_enabled()
    offload = training and getattr(cfg, "activation_offload", False)
    ctx = torch.autograd.graph.save_on_cpu(pin_memory=True) if offload else nullcontext()
    with ctx:
        if not full:
            return _run_range(blocks, 0, n, extra)(x)
        method = getattr(cfg, "recompute_method", "block") or "block"
        k = int(getattr(cfg, "recompute_num_layers", 0) or 0)
        if method == "uniform":
            k = max(k, 1)
            i = 0
            while i < n:
                x = _checkpointed(blocks, i, min(i + k, n), extra, x)
                i += k
            return x
        if method == "block":
            for i in range(n):
                if i < k:
                    x = _checkpointed(blocks, i, i + 1, extra, x)
                else:
                    x = blocks[i](x, *extra)
            return x
        raise ValueError(f"unknown recompute method {method!r}")
