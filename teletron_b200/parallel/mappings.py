"""Function-level split / gather mappings over a process group, with uneven chunk sizes and gradient scaling.

``split_forward_gather_backward(x, group, dim, split_sizes=None, grad_scale=None)`` keeps this rank's chunk of ``x``
along ``dim`` (backward: all ranks' gradient chunks concatenated) and ``gather_forward_split_backward(x, group, dim,
gather_sizes=None, grad_scale=None)`` is its inverse; ``grad_scale`` is ``"up"`` (multiply the gradient by the group
size), ``"down"`` (divide) or ``None`` / ``"none"``.  Same contract as the reference's mappings
(teletron/core/context_parallel/mappings.py:60-235).  Without explicit sizes a length that does not divide is spread
as evenly as possible (the first ``length % P`` ranks get one element more).  One autograd function serves both
directions, the collective is one ``all_gather`` of equal-sized padded chunks (so NCCL and gloo both take it, CPU
tensors included) instead of a list gather of ragged tensors.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def even_sizes(length: int, world: int) -> List[int]:
    base, rem = divmod(length, world)
    return [base + (1 if i < rem else 0) for i in range(world)]


def _scale(grad, mode, world):
    if mode == "up":
        return grad * world
    if mode == "down":
        return grad / world
    if mode in (None, "none"):
        return grad
    raise ValueError(f"grad_scale must be 'up', 'down' or None, got {mode!r}")


def _split(x, group, dim, sizes: Optional[Sequence[int]]):
    world = dist.get_world_size(group)
    if world == 1:
        return x
    sizes = list(sizes) if sizes else even_sizes(x.shape[dim], world)
    if len(sizes) != world or sum(sizes) != x.shape[dim]:
        raise ValueError(f"split sizes {sizes} do not cover length {x.shape[dim]} over {world} ranks")
    rank = dist.get_rank(group)
    return x.narrow(dim, sum(sizes[:rank]), sizes[rank]).contiguous()


def _gather(x, group, dim, sizes: Optional[Sequence[int]]):
    world = dist.get_world_size(group)
    if world == 1:
        return x
    rank = dist.get_rank(group)
    sizes = list(sizes) if sizes else [x.shape[dim]] * world
    if len(sizes) != world or sizes[rank] != x.shape[dim]:
        raise ValueError(f"gather sizes {sizes} disagree with this rank's length {x.shape[dim]}")
    longest = max(sizes)
    xm = x.movedim(dim, 0).contiguous()
    if xm.shape[0] < longest:
        xm = torch.cat([xm, xm.new_zeros((longest - xm.shape[0],) + tuple(xm.shape[1:]))], dim=0)
    out = xm.new_empty((world * longest,) + tuple(xm.shape[1:]))
    dist.all_gather_into_tensor(out, xm, group=group)
    parts = [out[i * longest: i * longest + sizes[i]] for i in range(world)]
    return torch.cat(parts, dim=0).movedim(0, dim).contiguous()


class _Mapping(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, sizes, grad_scale, split_forward):
        ctx.group, ctx.dim, ctx.sizes, ctx.grad_scale, ctx.split_forward = group, dim, sizes, grad_scale, split_forward
        return _split(x, group, dim, sizes) if split_forward else _gather(x, group, dim, sizes)

    @staticmethod
    def backward(ctx, g):
        g = _scale(g, ctx.grad_scale, dist.get_world_size(ctx.group))
        out = _gather(g, ctx.group, ctx.dim, ctx.sizes) if ctx.split_forward else _split(g, ctx.group, ctx.dim, ctx.sizes)
        return out, None, None, None, None, None


def split_forward_gather_backward(x, group=None, dim: int = -1, split_sizes: Optional[Sequence[int]] = None,
                                  grad_scale: Optional[str] = None):
    dim = dim % x.dim()
    if split_sizes is None and dist.get_world_size(group) > 1:
        split_sizes = even_sizes(x.shape[dim], dist.get_world_size(group))
    return _Mapping.apply(x, group, dim, split_sizes, grad_scale, True)


def gather_forward_split_backward(x, group=None, dim: int = -1, gather_sizes: Optional[Sequence[int]] = None,
                                  grad_scale: Optional[str] = None):
    return _Mapping.apply(x, group, dim % x.dim(), gather_sizes, grad_scale, False)
