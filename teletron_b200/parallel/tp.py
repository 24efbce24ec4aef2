"""Tensor parallelism with sequence-sharded activations (Megatron "TP + SP" layout).

The reference builds TP groups but shards no layer (teletron/core/parallel_state.py:481-491;
no ColumnParallel/RowParallel layer exists in its models), so this is new functionality:

  ColumnParallelLinear   y[:, shard] = all_gather_rows(x) @ W[shard, :]^T       (AG -> GEMM)
  RowParallelLinear      y_rows(rank) = reduce_scatter_rows(x[:, shard] @ W[:, shard]^T) + b   (GEMM -> RS)

Activations between TP regions are sharded along tokens (rows), so LayerNorm / AdaLN / residual
work on 1/T of the rows.  Backward of the all-gather is a reduce-scatter and vice versa.
Weights are stored as shards; ``tp_shard_state_dict`` / ``tp_merge_state_dicts`` convert between a
full state dict and per-rank shards (checkpoint files ``mp_rank_XX``).
The collectives here are torch.distributed (NCCL / gloo); GEMMs are the tcgen05 kernels.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops


def _ag_rows(x, group, world):
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _rs_rows(x, group, world):
    assert x.shape[0] % world == 0, "rows must divide by the tensor-parallel size"
    out = torch.empty((x.shape[0] // world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x.contiguous(), op=dist.ReduceOp.SUM, group=group)
    else:  # gloo has no reduce-scatter: all-reduce and keep our slice
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        r = dist.get_rank(group)
        out.copy_(y[r * out.shape[0]:(r + 1) * out.shape[0]])
    return out


class GatherRows(torch.autograd.Function):
    """all-gather along rows; backward reduce-scatters (sum) the gradient."""

    @staticmethod
    def forward(ctx, x, group, world):
        ctx.group, ctx.world = group, world
        return _ag_rows(x, group, world)

    @staticmethod
    def backward(ctx, g):
        return _rs_rows(g, ctx.group, ctx.world), None, None


class ReduceScatterRows(torch.autograd.Function):
    """reduce-scatter (sum) along rows; backward all-gathers the gradient."""

    @staticmethod
    def forward(ctx, x, group, world):
        ctx.group, ctx.world = group, world
        return _rs_rows(x, group, world)

    @staticmethod
    def backward(ctx, g):
        return _ag_rows(g, ctx.group, ctx.world), None, None


class GatherRowsKeepLocalGrad(torch.autograd.Function):
    """all-gather along rows for a result that every rank then uses identically (the model output that
    feeds a replicated loss): backward keeps this rank's rows of the gradient, no reduction."""

    @staticmethod
    def forward(ctx, x, group, world, rank):
        ctx.meta = (rank, x.shape[0])
        return _ag_rows(x, group, world)

    @staticmethod
    def backward(ctx, g):
        rank, n = ctx.meta
        return g[rank * n:(rank + 1) * n].contiguous(), None, None, None


class TPContext:
    def __init__(self, group=None, size: int = 1, rank: int = 0):
        self.group, self.size, self.rank = group, size, rank

    def gather_rows(self, x):
        return GatherRows.apply(x, self.group, self.size) if self.size > 1 else x

    def gather_rows_for_output(self, x):
        return GatherRowsKeepLocalGrad.apply(x, self.group, self.size, self.rank) if self.size > 1 else x

    def reduce_scatter_rows(self, x):
        return ReduceScatterRows.apply(x, self.group, self.size) if self.size > 1 else x

    def split_rows(self, x):
        if self.size == 1:
            return x
        n = x.shape[0] // self.size
        return x.narrow(0, self.rank * n, n)


class ColumnParallelLinear(nn.Module):
    """Holds rows [rank*N/T, (rank+1)*N/T) of a [N, K] weight. Input: row-sharded [M/T, K]."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = True):
        super().__init__()
        assert out_features % tp.size == 0
        self.tp, self.in_features, self.out_features = tp, in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // tp.size, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features // tp.size)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        self.shard_dim = 0

    def forward(self, x_rows, act=None, gathered: bool = False):
        x = x_rows if gathered else self.tp.gather_rows(x_rows)
        return ops.linear(x, self.weight, self.bias, act)


class RowParallelLinear(nn.Module):
    """Holds columns [rank*K/T, (rank+1)*K/T) of a [N, K] weight. Output: row-sharded [M/T, N]."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = True):
        super().__init__()
        assert in_features % tp.size == 0
        self.tp, self.in_features, self.out_features = tp, in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp.size))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        self.shard_dim = 1

    def forward(self, x_cols):
        y = ops.linear(x_cols, self.weight, None)
        y = self.tp.reduce_scatter_rows(y)
        if self.bias is not None:
            y = y + self.bias
        return y


# ------------------------------------------------------------------------------ checkpoints
def _slice_groups(v, d, groups, rank, world):
    """Slice dim ``d`` of ``v`` per group: dim d is a concatenation of ``groups`` widths, each sharded."""
    parts, pos = [], 0
    for g in groups:
        n = g // world
        parts.append(v.narrow(d, pos + rank * n, n))
        pos += g
    return torch.cat(parts, dim=d).contiguous()


def tp_shard_state_dict(full: Dict[str, torch.Tensor], shard_dims: Dict[str, object], rank: int, world: int):
    """Slice every tensor named in ``shard_dims`` (name -> dim, or (dim, column groups)) for ``rank``;
    others are copied."""
    out = {}
    for k, v in full.items():
        d = shard_dims.get(k)
        if d is None or world == 1:
            out[k] = v
        elif isinstance(d, tuple):
            out[k] = _slice_groups(v, d[0], d[1], rank, world)
        else:
            n = v.shape[d] // world
            out[k] = v.narrow(d, rank * n, n).contiguous()
    return out


def tp_merge_state_dicts(shards: List[Dict[str, torch.Tensor]], shard_dims: Dict[str, int]):
    out = {}
    world = len(shards)
    for k in shards[0]:
        d = shard_dims.get(k)
        if d is None or world == 1:
            out[k] = shards[0][k]
        elif isinstance(d, tuple):
            dim, groups = d
            pieces, pos = [], 0
            for g in groups:
                n = g // world
                pieces.extend(s[k].narrow(dim, pos, n) for s in shards)
                pos += n
            out[k] = torch.cat(pieces, dim=dim)
        else:
            out[k] = torch.cat([s[k] for s in shards], dim=d)
    return out


def tp_shard_dims(module: nn.Module) -> Dict[str, int]:
    dims = {}
    for name, m in module.named_modules():
        if isinstance(m, (ColumnParallelLinear, RowParallelLinear)):
            groups = getattr(m, "col_groups", None)
            dims[f"{name}.weight"] = (m.shard_dim, tuple(groups)) if groups else m.shard_dim
            if isinstance(m, ColumnParallelLinear) and m.bias is not None:
                dims[f"{name}.bias"] = 0
    return dims
