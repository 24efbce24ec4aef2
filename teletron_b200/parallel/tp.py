"""Tensor parallelism with sequence-sharded activations (Megatron "TP + SP" layout).

The reference builds TP groups but shards no layer (teletron/core/parallel_state.py:481-491;
no ColumnParallel/RowParallel layer exists in its models), so this is new functionality:

  ColumnParallelLinear   y[:, shard] = all_gather_rows(x) @ W[shard, :]^T       (AG -> GEMM)
  RowParallelLinear      y_rows(rank) = reduce_scatter_rows(x[:, shard] @ W[:, shard]^T) + b   (GEMM -> RS)

Activations between TP regions are sharded along tokens (rows), so LayerNorm / AdaLN / residual
work on 1/T of the rows.  Backward of the all-gather is a reduce-scatter and vice versa.
Weights are stored as shards; ``tp_shard_state_dict`` / ``tp_merge_state_dicts`` convert between a
full state dict and per-rank shards (checkpoint files ``mp_rank_XX``).
The collectives are torch.distributed (NCCL / gloo) by default; when the TP group shares one NVLink box the trainer
attaches a ``FusedTP`` and the linears run the all-gather inside the GEMM's TMA loads and the reduce-scatter
inside its epilogue (csrc/gemm.cu).  GEMMs are the tcgen05 kernels either way.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..utils.nvtx import nvtx_range


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


class FusedTP:
    """Peer-memory buffers and call order for the fused tensor-parallel kernels of one TP group on one box:

      all-gather -> GEMM    each rank copies its rows into a symmetric buffer, a device barrier follows, and one
                            GEMM kernel pulls the remote segments over NVLink with its copier warps while its
                            tensor-core tiles start on the local segment (``ops.gemm_ag_gather``)
      GEMM -> reduce-scatter  the GEMM epilogue stores each tile of partial sums into the staging buffer of the rank
                            that owns the rows (``ops.gemm_rs_scatter``); after a barrier every rank sums its
                            ``world`` slots (``ops.tp_reduce_rows``)

    Both buffers are double-buffered: the barrier of call n+1 is stream-ordered behind each rank's reads of call n,
    so buffer n % 2 may be overwritten again in call n+2.  Every rank must issue the same calls in the same order.
    """

    def __init__(self, arena):
        self.arena = arena
        self.world, self.rank = arena.world, arena.rank
        self._x = [None, None]
        self._st = [None, None]
        self._x_cap = 0
        self._st_cap = 0
        self._n_ag = 0
        self._n_rs = 0
        self._ag_flags = None      # one flag per 128-row block of the gathered operand, epoch-valued
        self._ag_epoch = 0

    def _x_buf(self, numel):
        if numel > self._x_cap:  # collective: every rank grows at the same call
            self._x = [self.arena.alloc(numel, torch.bfloat16) for _ in range(2)]
            self._x_cap = numel
        self._n_ag += 1
        return self._x[self._n_ag & 1]

    def _st_buf(self, numel):
        if numel > self._st_cap:
            self._st = [self.arena.alloc(numel, torch.bfloat16) for _ in range(2)]
            self._st_cap = numel
        self._n_rs += 1
        return self._st[self._n_rs & 1]

    def ag_gemm(self, x_rows, w, *, b_mn=False, bias=None, epi=0, want_aux=False):
        """epilogue(all_gather_rows(x_rows) @ W^T) in one kernel: x_rows [rows, k] bf16, W [n, k] (or [k, n] when
        b_mn).  Returns (y, pre-activation or None, gathered x or None).

        Every rank puts its rows into a symmetric buffer; after a device barrier the GEMM kernel itself gathers the
        operand (``ops.gemm_ag_gather``, csrc/gemm2.cu): two copier warps per CTA pull the segments, 128 rows at a
        time, into a local gathered matrix and flag them, the tiles of the local segment are multiplied first and
        the others as their rows land, so each remote element crosses NVLink once and the gathered matrix is left
        for the weight gradient.  Outputs narrower than 256 columns (or fewer than 256 rows) use ``ops.gemm_ag``,
        whose TMA loads read the peers' buffers directly (no gathered copy; fine when there are few column tiles)."""
        rows, k = x_rows.shape
        buf = self._x_buf(rows * k)
        mine = buf.tensor[: rows * k].view(rows, k)
        mine.copy_(x_rows)
        self.arena.barrier(0)
        n = w.shape[1] if b_mn else w.shape[0]
        if n >= 256 and rows * self.world >= 256:
            with nvtx_range("ag_gemm"):
                blocks = (rows * self.world + 127) // 128
                if self._ag_flags is None or self._ag_flags.numel() < blocks:
                    self._ag_flags = torch.zeros(blocks, dtype=torch.int32, device=x_rows.device)
                    self._ag_epoch = 0
                self._ag_epoch = (self._ag_epoch % 0x7FFFFFF0) + 1
                y, aux, gathered = ops.gemm_ag_gather(buf.peer_ptrs, rows, k, w, self._ag_flags, self._ag_epoch,
                                                      self.rank, b_mn=b_mn, bias=bias, epi=epi, want_aux=want_aux,
                                                      device=x_rows.device)
            return y, aux, gathered
        res = ops.gemm_ag(buf.peer_ptrs, rows, k, w, b_mn=b_mn, bias=bias, epi=epi, want_aux=want_aux,
                          device=x_rows.device)
        return (res[0], res[1], None) if want_aux else (res, None, None)

    def gemm_rs(self, x, w, *, b_mn=False):
        """reduce_scatter_rows(x @ W^T): x [world * rows, k]; returns this rank's [rows, n] of the sum."""
        m = x.shape[0]
        assert m % self.world == 0, "rows must divide by the tensor-parallel size"
        rows = m // self.world
        n = w.shape[1] if b_mn else w.shape[0]
        st = self._st_buf(self.world * rows * n)
        ops.gemm_rs_scatter(x, w, st.peer_ptrs, rows, self.rank, b_mn=b_mn)
        self.arena.barrier(0)
        return ops.tp_reduce_rows(st.tensor, self.world, rows, n)


class _FusedColumnLinear(torch.autograd.Function):
    """act(all_gather_rows(x) @ W^T + b) with the gather overlapped with (or inside) the GEMM; backward
    reduce-scatters dX through the GEMM epilogue.  The weight gradient reuses the gathered activations."""

    @staticmethod
    def forward(ctx, x_rows, w, b, act, tp):
        from ..ops.linear import _ACT

        need_pre = act is not None
        y, pre, gathered = tp.fused.ag_gemm(x_rows, w, bias=b, epi=_ACT[act], want_aux=need_pre)
        # the gathered activations are kept for the weight gradient when the gather produced them
        ctx.save_for_backward(x_rows if gathered is None else gathered, w, pre)
        ctx.have_gathered = gathered is not None
        ctx.act, ctx.tp, ctx.bias_ref, ctx.w_param = act, tp, b, w
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.linear import _bias_grad, _weight_grad, act_bwd

        x_rows, w, pre = ctx.saved_tensors
        tp = ctx.tp
        if dy.stride(1) != 1:
            dy = dy.contiguous()
        if ctx.act is not None:
            dy = act_bwd(dy, pre, ctx.act)
        dx = tp.fused.gemm_rs(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            xg = x_rows if ctx.have_gathered else _ag_rows(x_rows, tp.group, tp.size)
            dw = _weight_grad(dy, xg, w, ctx.w_param)
        db = _bias_grad(dy, ctx.bias_ref) if (ctx.bias_ref is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None


class _FusedRowLinear(torch.autograd.Function):
    """reduce_scatter_rows(x @ W^T) with the scatter inside the GEMM epilogue; backward gathers dY inside the
    dgrad GEMM."""

    @staticmethod
    def forward(ctx, x_cols, w, tp):
        ctx.save_for_backward(x_cols, w)
        ctx.tp, ctx.w_param = tp, w
        return tp.fused.gemm_rs(x_cols, w)

    @staticmethod
    def backward(ctx, dy_rows):
        from ..ops.linear import _weight_grad

        x_cols, w = ctx.saved_tensors
        tp = ctx.tp
        if dy_rows.stride(1) != 1:
            dy_rows = dy_rows.contiguous()
        dx, dyg = None, None
        if ctx.needs_input_grad[0]:
            dx, _, dyg = tp.fused.ag_gemm(dy_rows, w, b_mn=True)
        dw = None
        if ctx.needs_input_grad[1]:
            if dyg is None:
                dyg = _ag_rows(dy_rows, tp.group, tp.size)
            dw = _weight_grad(dyg, x_cols, w, ctx.w_param)
        return dx, dw, None


class TPContext:
    def __init__(self, group=None, size: int = 1, rank: int = 0):
        self.group, self.size, self.rank = group, size, rank
        self.fused: Optional[FusedTP] = None  # set by the trainer when the group shares one NVLink box

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


def _init_shard(out_features: int, in_features: int, dim: int, tp: "TPContext") -> torch.Tensor:
    """This rank's slice along ``dim`` of a freshly initialised FULL [out, in] weight.  Every tensor-parallel rank
    draws the same full matrix from the shared random stream (all ranks are seeded alike) and keeps its own
    slice: the shards differ between ranks, the merged weight is distributed exactly like the unsharded layer
    (fan-in of the full layer), and the random stream stays in step across ranks."""
    full = torch.empty(out_features, in_features)
    nn.init.kaiming_uniform_(full, a=math.sqrt(5))
    n = full.shape[dim] // tp.size
    return full.narrow(dim, tp.rank * n, n).clone()


class ColumnParallelLinear(nn.Module):
    """Holds rows [rank*N/T, (rank+1)*N/T) of a [N, K] weight. Input: row-sharded [M/T, K]."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = True):
        super().__init__()
        assert out_features % tp.size == 0
        self.tp, self.in_features, self.out_features = tp, in_features, out_features
        self.weight = nn.Parameter(_init_shard(out_features, in_features, 0, tp))
        self.bias = nn.Parameter(torch.zeros(out_features // tp.size)) if bias else None
        self.shard_dim = 0

    def forward(self, x_rows, act=None, gathered: bool = False):
        if (not gathered and self.tp.size > 1 and self.tp.fused is not None and x_rows.is_cuda
                and x_rows.dim() == 2 and self.weight.shape[0] > 64):
            return _FusedColumnLinear.apply(x_rows, self.weight, self.bias, act, self.tp)
        x = x_rows if gathered else self.tp.gather_rows(x_rows)
        return ops.linear(x, self.weight, self.bias, act)


class FusedColumnParallel(ColumnParallelLinear):
    """Several column-parallel projections of the same input as ONE GEMM (q / k / v): the local weight is
    ``[n * out / T, in]`` with one row block per projection, so a single all-gather -> GEMM serves all of them.  In
    state dicts the projections appear under their own names (``names``: sibling keys ``<name>.weight`` /
    ``<name>.bias`` beside this module's key), each holding this rank's shard, so checkpoints keep the per-projection
    layout of the unfused model.  The module that owns this one calls ``install_state_hooks(owner, attribute)``:
    ``load_state_dict`` hands a child only the keys under its own prefix, so the renaming has to happen one level up."""

    def __init__(self, in_features: int, out_features: int, names, tp: TPContext, bias: bool = True):
        nn.Module.__init__(self)
        assert out_features % tp.size == 0
        self.tp, self.in_features, self.out_features, self.names = tp, in_features, out_features, tuple(names)
        self.out_local = out_features // tp.size
        self.weight = nn.Parameter(torch.cat([_init_shard(out_features, in_features, 0, tp) for _ in self.names]))
        self.bias = nn.Parameter(torch.zeros(len(self.names) * self.out_local)) if bias else None
        self.shard_dim = 0
        self.col_groups = tuple(out_features for _ in self.names)     # of the merged (all TP ranks) weight

    @staticmethod
    def install_state_hooks(owner: nn.Module, attr: str):
        def save_hook(module, state, prefix, _local):
            fp = getattr(module, attr)
            for kind in ("weight", "bias"):
                key = f"{prefix}{attr}.{kind}"
                if key in state:
                    t = state.pop(key)
                    for i, n in enumerate(fp.names):
                        state[f"{prefix}{n}.{kind}"] = t[i * fp.out_local:(i + 1) * fp.out_local]
            return state

        def load_hook(module, state, prefix, *_):
            fp = getattr(module, attr)
            for kind in ("weight", "bias"):
                keys = [f"{prefix}{n}.{kind}" for n in fp.names]
                if all(k in state for k in keys):
                    state[f"{prefix}{attr}.{kind}"] = torch.cat([state.pop(k) for k in keys], dim=0)

        owner._register_state_dict_hook(save_hook)
        owner.register_load_state_dict_pre_hook(load_hook)

    def split(self, y):
        """The projections' column blocks of the fused output."""
        n = self.out_local
        return tuple(y[:, i * n:(i + 1) * n] for i in range(len(self.names)))


class RowParallelLinear(nn.Module):
    """Holds columns [rank*K/T, (rank+1)*K/T) of a [N, K] weight. Output: row-sharded [M/T, N]."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = True):
        super().__init__()
        assert in_features % tp.size == 0
        self.tp, self.in_features, self.out_features = tp, in_features, out_features
        self.weight = nn.Parameter(_init_shard(out_features, in_features, 1, tp))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.shard_dim = 1

    def forward(self, x_cols):
        if (self.tp.size > 1 and self.tp.fused is not None and x_cols.is_cuda and x_cols.dim() == 2
                and self.weight.shape[0] > 64):
            y = _FusedRowLinear.apply(x_cols, self.weight, self.tp)
        else:
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


def tp_shard_dims(module: nn.Module, params: bool = False) -> Dict[str, object]:
    """Which tensors are tensor-parallel shards, and along which dim (or ``(dim, column groups)``).  Keys are
    state-dict names by default; with ``params`` they are parameter names (they differ for fused projections,
    which state dicts list per projection)."""
    dims = {}
    for name, m in module.named_modules():
        if isinstance(m, FusedColumnParallel):
            if params:
                dims[f"{name}.weight"] = (0, m.col_groups)
                if m.bias is not None:
                    dims[f"{name}.bias"] = (0, m.col_groups)
            else:
                parent = name.rsplit(".", 1)[0] + "." if "." in name else ""
                for n in m.names:
                    dims[f"{parent}{n}.weight"] = 0
                    if m.bias is not None:
                        dims[f"{parent}{n}.bias"] = 0
        elif isinstance(m, (ColumnParallelLinear, RowParallelLinear)):
            groups = getattr(m, "col_groups", None)
            dims[f"{name}.weight"] = (m.shard_dim, tuple(groups)) if groups else m.shard_dim
            if isinstance(m, ColumnParallelLinear) and m.bias is not None:
                dims[f"{name}.bias"] = 0
    return dims
