"""Ulysses context parallelism: sequence split/gather with padding and the seq<->head
all-to-all around attention.

Functional counterpart of the reference mixin and mappings
(teletron/core/context_parallel/context_parallel_mixin.py:21-131,
teletron/core/context_parallel/mappings.py:9-236) with instance state instead of class
attributes.  The sequence is zero-padded at the tail to a multiple of the group size; the
padded keys are masked inside the attention kernel (key-length argument) rather than stripped
and re-added around it.  Heads that do not divide the group size are padded with zero heads.
This module is the torch.distributed (NCCL or gloo) path; the fused peer-memory kernels in
``parallel.fused_ulysses`` replace the all-to-all copies on NVLink-connected GPUs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops


def _all_to_all(x: torch.Tensor, group) -> torch.Tensor:
    """x: [P, ...] contiguous; returns [P, ...] where out[p] is what rank p sent to this rank."""
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)  # NCCL on GPU, gloo on CPU
    return out


class _SeqToHead(torch.autograd.Function):
    """[B, S_l, H, D] -> [B, P*S_l, H/P, D]; backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, group, P):
        ctx.group, ctx.P = group, P
        return _seq_to_head(x, group, P)

    @staticmethod
    def backward(ctx, g):
        return _head_to_seq(g.contiguous(), ctx.group, ctx.P), None, None


class _HeadToSeq(torch.autograd.Function):
    """[B, P*S_l, H/P, D] -> [B, S_l, H, D]; backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, group, P):
        ctx.group, ctx.P = group, P
        return _head_to_seq(x, group, P)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_head(g.contiguous(), ctx.group, ctx.P), None, None


def _seq_to_head(x, group, P):
    B, Sl, H, D = x.shape
    Hl = H // P
    send = x.reshape(B, Sl, P, Hl, D).permute(2, 0, 1, 3, 4).contiguous()
    recv = _all_to_all(send, group)  # [P, B, Sl, Hl, D]
    return recv.permute(1, 0, 2, 3, 4).reshape(B, P * Sl, Hl, D)


def _head_to_seq(x, group, P):
    B, S, Hl, D = x.shape
    Sl = S // P
    send = x.reshape(B, P, Sl, Hl, D).permute(1, 0, 2, 3, 4).contiguous()
    recv = _all_to_all(send, group)  # [P, B, Sl, Hl, D]
    return recv.permute(1, 2, 0, 3, 4).reshape(B, Sl, P * Hl, D)


class _GatherTokens(torch.autograd.Function):
    """all-gather along tokens; backward keeps the local slice (no scaling), which is what a loss
    evaluated identically on every rank needs (context_parallel_mixin.py:47-52)."""

    @staticmethod
    def forward(ctx, x, group, P, rank):
        ctx.meta = (P, rank, x.shape[1])
        parts = [torch.empty_like(x) for _ in range(P)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=1)

    @staticmethod
    def backward(ctx, g):
        P, rank, Sl = ctx.meta
        return g[:, rank * Sl:(rank + 1) * Sl].contiguous(), None, None, None


class UlyssesContext:
    """Holds the CP group and the current sequence bookkeeping."""

    def __init__(self, group=None, size: Optional[int] = None, rank: Optional[int] = None):
        self.group = group
        self.size = size if size is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.seq_len = None      # un-padded global sequence length of the current batch
        self.local_len = None
        self.fused = None        # parallel.fused_ulysses.FusedUlysses when peer-memory kernels are enabled

    # ---- sequence split / gather -------------------------------------------------------
    def padded_len(self, S: int) -> int:
        return (S + self.size - 1) // self.size * self.size

    def split_tokens(self, x):
        """[B, S, ...] -> local [B, ceil(S/P), ...] chunk (tail zero-padded). Differentiable."""
        S = x.shape[1]
        Sp = self.padded_len(S)
        self.seq_len, self.local_len = S, Sp // self.size
        if Sp != S:
            pad = [0, 0] * (x.dim() - 2) + [0, Sp - S]
            x = F.pad(x, pad)
        return x.narrow(1, self.rank * self.local_len, self.local_len)

    def split_rows(self, t):
        """Split a per-token table [S, ...] the same way (no batch dim)."""
        return self.split_tokens(t.unsqueeze(0)).squeeze(0).contiguous()

    def gather_tokens(self, x, S: Optional[int] = None):
        """[B, S_l, ...] -> [B, S, ...] on every rank; padding removed."""
        S = S if S is not None else self.seq_len
        full = _GatherTokens.apply(x, self.group, self.size, self.rank)
        return full[:, :S]

    # ---- attention -----------------------------------------------------------------------
    def attention(self, q, k, v, scale=None):
        """q,k,v: local [B, S_l, H, D]; returns local [B, S_l, H, D] of full-sequence attention."""
        P = self.size
        B, Sl, H, D = q.shape
        Hp = (H + P - 1) // P * P
        if Hp != H:
            q, k, v = (F.pad(t, (0, 0, 0, Hp - H)) for t in (q, k, v))
        qh = _SeqToHead.apply(q.contiguous(), self.group, P)
        kh = _SeqToHead.apply(k.contiguous(), self.group, P)
        vh = _SeqToHead.apply(v.contiguous(), self.group, P)
        kv_lens = None
        if self.seq_len is not None and self.seq_len != P * Sl:
            kv_lens = torch.full((B,), self.seq_len, dtype=torch.int32, device=q.device)
        oh = ops.attention(qh, kh, vh, scale, kv_lens)
        o = _HeadToSeq.apply(oh.contiguous(), self.group, P)
        return o[:, :, :H] if Hp != H else o

    # ---- the reference mixin's spellings (teletron/core/context_parallel/context_parallel_mixin.py:39-125) -------
    def split_input(self, x, dim: int = 1):
        """Pad ``x`` along ``dim`` to a multiple of the group size and keep this rank's chunk (backward gathers)."""
        if dim == 1:
            return self.split_tokens(x)
        return self.split_tokens(x.movedim(dim, 1)).movedim(1, dim)

    def gather_output(self, output, dim: int = 1):
        """Inverse of ``split_input``: all ranks' chunks concatenated along ``dim``, padding removed."""
        if dim == 1:
            return self.gather_tokens(output)
        return self.gather_tokens(output.movedim(dim, 1)).movedim(1, dim)

    def forward_attn(self, q, k, v, num_heads: int):
        """q, k, v: local ``[B, S_l, H*D]``; returns ``[B, S_l, H*D]`` of attention over the whole sequence."""
        B, Sl, C = q.shape
        D = C // num_heads
        o = self.attention(q.view(B, Sl, num_heads, D), k.view(B, Sl, num_heads, D), v.view(B, Sl, num_heads, D))
        return o.reshape(B, Sl, C)
