"""Flat parameter / gradient buffers, data-parallel gradient reduction and the (optionally
sharded) AdamW optimizer with fp32 master weights.

What the reference spreads over its DDP wrapper, bucketed grad buffer and Megatron's
optimizers (teletron/core/distributed/distributed_data_parallel.py:14-298,
teletron/core/distributed/param_and_grad_buffer.py:31-520, teletron/train/lr_scheduler.py:423-509)
is one object here:

  * ``ParamBuffer`` re-points every parameter into one contiguous bf16 buffer and gives it a
    ``main_grad`` view into one contiguous fp32 buffer.  Weight gradients are accumulated into
    ``main_grad`` by the wgrad GEMM epilogue; small parameters (biases, norms, modulation) get
    ordinary ``.grad`` tensors that ``collect_grads`` folds in.  Parameters with weight decay
    come first, the rest after, each region padded so it splits evenly across ranks.
  * ``DistributedOptimizer`` reduces gradients over the DP x CP group — a reduce-scatter
    straight on the fp32 buffer when sharded (the reference all-reduces through a 400 MB fp32
    staging copy, param_and_grad_buffer.py:128-148) — computes the global gradient norm, runs
    the fused AdamW kernel on the owned shard and all-gathers the bf16 parameters.
  * gradient scale: all parameter gradients are partial sums over the CP group (the loss is
    normalised by the full token count), so the reduction is a plain sum and the scale is
    ``1 / dp`` (times ``1 / num_microbatches`` folded into the loss).
"""
from __future__ import annotations

import contextlib
import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops

_ALIGN = 8  # elements; keeps every parameter 16-byte aligned in the bf16 buffer


def _no_weight_decay(name: str, p: torch.Tensor) -> bool:
    """Megatron's default grouping: biases and 1-D parameters are not decayed."""
    return name.endswith(".bias") or p.dim() == 1


class ParamBuffer:
    def __init__(self, module: torch.nn.Module, shard_world: int = 1, grad_dtype=torch.float32, arena=None):
        """``arena``: a ``dist.SymmetricArena``; when given, both flat buffers live in symmetric peer
        memory so the fused reduce-scatter / AdamW / all-gather kernels can reach every rank's copy."""
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        assert named, "module has no trainable parameters"
        dev = named[0][1].device
        self.param_dtype = named[0][1].dtype
        self.grad_dtype = grad_dtype
        decay = [(n, p) for n, p in named if not _no_weight_decay(n, p)]
        nodecay = [(n, p) for n, p in named if _no_weight_decay(n, p)]
        self.region_align = max(shard_world, 1) * 4 * _ALIGN
        self.index: Dict[str, Tuple[int, int, torch.Size]] = {}
        off = 0
        for n, p in decay:
            self.index[n] = (off, p.numel(), p.shape)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.decay_end = (off + self.region_align - 1) // self.region_align * self.region_align
        off = self.decay_end
        for n, p in nodecay:
            self.index[n] = (off, p.numel(), p.shape)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.numel = (off + self.region_align - 1) // self.region_align * self.region_align
        self.arena = arena
        self.symm_params = self.symm_grads = None
        if arena is not None:
            self.symm_params = arena.alloc(self.numel, self.param_dtype)
            self.symm_grads = arena.alloc(self.numel, grad_dtype)
            self.params, self.grads = self.symm_params.tensor, self.symm_grads.tensor
            self.params.zero_()
            self.grads.zero_()
        else:
            self.params = torch.zeros(self.numel, dtype=self.param_dtype, device=dev)
            self.grads = torch.zeros(self.numel, dtype=grad_dtype, device=dev)
        self.named = named
        for n, p in named:
            o, cnt, shape = self.index[n]
            self.params[o:o + cnt].copy_(p.data.reshape(-1))
            p.data = self.params[o:o + cnt].view(shape)
            p.main_grad = self.grads[o:o + cnt].view(shape)
            p.grad_written = False

    def zero_grads(self):
        self.grads.zero_()
        for _, p in self.named:
            p.grad = None
            p.grad_written = False

    def collect_grads(self):
        """Fold autograd ``.grad`` tensors (parameters not written by a wgrad epilogue) into main_grad."""
        for _, p in self.named:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    def runs_excluding(self, names) -> List[Tuple[int, int]]:
        """Contiguous (start, end) element ranges covering every parameter NOT in ``names``."""
        spans = sorted((o, o + (n + _ALIGN - 1) // _ALIGN * _ALIGN) for k, (o, n, _) in self.index.items()
                       if k not in names)
        runs: List[Tuple[int, int]] = []
        for s, e in spans:
            if runs and runs[-1][1] == s:
                runs[-1] = (runs[-1][0], e)
            else:
                runs.append((s, e))
        return runs

    def regions(self) -> List[Tuple[int, int, bool]]:
        """(start, end, weight_decay?) of the two regions."""
        out = []
        if self.decay_end > 0:
            out.append((0, self.decay_end, True))
        if self.numel > self.decay_end:
            out.append((self.decay_end, self.numel, False))
        return out


class DistributedOptimizer:
    """AdamW over a ParamBuffer. ``group``: the DP x CP process group (None = single process).

    ``sharded=True`` is the ZeRO-1 layout (``--use-distributed-optimizer``): each rank keeps fp32
    master / m / v for 1/world of each region.  ``grad_scale`` is applied to the summed gradient
    (use 1/dp).  ``step()`` returns (ok, grad_norm, None) like Megatron's optimizers.
    """

    def __init__(self, buf: ParamBuffer, group=None, *, lr=1e-4, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.01, clip_grad=0.0, sharded=False, grad_scale=1.0, tp_group=None,
                 tp_sharded_names=()):
        """``tp_group`` / ``tp_sharded_names``: under tensor parallelism the gradients of parameters
        that are replicated across the TP group (everything not in ``tp_sharded_names``) are partial
        sums over that group's row shards and are all-reduced over it before the DP x CP reduction."""
        self.buf, self.group = buf, group
        self.tp_group = tp_group
        self.tp_runs = buf.runs_excluding(set(tp_sharded_names)) if tp_group is not None else []
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.sharded = bool(sharded) and self.world > 1
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.clip_grad, self.grad_scale = clip_grad, grad_scale
        self.step_count = 0
        self.param_groups = [dict(lr=lr, weight_decay=weight_decay)]  # scheduler-facing view
        self.shards: List[Tuple[int, int, bool]] = []
        for s, e, wd in buf.regions():
            if self.sharded:
                n = (e - s) // self.world
                self.shards.append((s + self.rank * n, s + (self.rank + 1) * n, wd))
            else:
                self.shards.append((s, e, wd))
        dev = buf.params.device
        self.master = [buf.params[s:e].float().clone() for s, e, _ in self.shards]
        self.exp_avg = [torch.zeros(e - s, dtype=torch.float32, device=dev) for s, e, _ in self.shards]
        self.exp_avg_sq = [torch.zeros(e - s, dtype=torch.float32, device=dev) for s, e, _ in self.shards]
        self._shard_grads: List[Optional[torch.Tensor]] = [None] * len(self.shards)
        # fused path: peer-memory reduce-scatter + AdamW + parameter scatter (csrc/comm.cu)
        self.fused = bool(self.sharded and buf.arena is not None and buf.grads.dtype == torch.float32)
        self.log_num_zeros = False
        self._reduced = None
        self.last_path = "nccl"

    # ------------------------------------------------------------------ gradient sync
    def reduce_gradients(self):
        """Sum gradients over the group; afterwards ``_shard_grads`` holds this rank's fp32 slices."""
        self.buf.collect_grads()
        g = self.buf.grads
        for s_, e_ in self.tp_runs:
            dist.all_reduce(g[s_:e_], op=dist.ReduceOp.SUM, group=self.tp_group)
        if self.fused:
            self._shard_grads = ["fused"] * len(self.shards)  # reduction happens inside step()
            return
        if self.world > 1:
            if self.sharded:
                for i, ((s, e, _), (rs, re, _)) in enumerate(zip(self.shards, self.buf.regions())):
                    out = g[s:e]
                    dist.reduce_scatter_tensor(out, g[rs:re], op=dist.ReduceOp.SUM, group=self.group)
            else:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)
        for i, (s, e, _) in enumerate(self.shards):
            self._shard_grads[i] = g[s:e]

    def _global_grad_norm(self) -> torch.Tensor:
        ss = None
        for gsh in self._shard_grads:
            t = ops.grad_norm(gsh.float() if gsh.dtype != torch.float32 else gsh)[2]
            ss = t if ss is None else ss + t
        if self.sharded:
            dist.all_reduce(ss, op=dist.ReduceOp.SUM, group=self.group)
        return ss.sqrt() * self.grad_scale

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def _fused_step(self):
        """K-DP-RS-ADAMW: barrier, pull-reduce of the owned shard from every peer, global norm, AdamW
        and bf16 parameter scatter to every peer, barrier."""
        from ..ops import _lib

        L = _lib.lib()
        buf, arena = self.buf, self.buf.arena
        dev = buf.params.device
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        wd_base = self.param_groups[0]["weight_decay"]
        blocks = L.tt_comm_blocks()
        need_clip = bool(self.clip_grad and self.clip_grad > 0)
        partials = torch.zeros((len(self.shards), blocks), dtype=torch.float32, device=dev)
        if need_clip and self._reduced is None:
            self._reduced = [torch.empty(e - s, dtype=torch.float32, device=dev) for s, e, _ in self.shards]
        arena.barrier(0)  # every rank's backward (its writes into its gradient buffer) is complete

        def launch(mode, i, coef):
            s, e, wd = self.shards[i]
            rc = L.tt_dp_shard_step(
                _lib.c_int(mode), buf.symm_grads.c_ptrs(), buf.symm_params.c_ptrs(), _lib.c_int(self.world),
                _lib.c_int(self.rank), _lib.c_ll(s), _lib.c_ll(e - s),
                _lib.ptr(self._reduced[i] if self._reduced is not None else None), _lib.ptr(self.master[i]),
                _lib.ptr(self.exp_avg[i]), _lib.ptr(self.exp_avg_sq[i]), _lib.c_float(self.grad_scale),
                _lib.ptr(coef), _lib.c_float(lr), _lib.c_float(self.betas[0]), _lib.c_float(self.betas[1]),
                _lib.c_float(self.eps), _lib.c_float(wd_base if wd else 0.0), _lib.c_int(self.step_count),
                _lib.ptr(partials[i]), _lib.stream())
            _lib.check(rc, "tt_dp_shard_step")

        for i in range(len(self.shards)):
            launch(0 if need_clip else 2, i, None)
        ss = partials.sum()
        dist.all_reduce(ss, op=dist.ReduceOp.SUM, group=self.group)
        norm = ss.sqrt() * self.grad_scale
        zeros = None
        if self.log_num_zeros and need_clip:      # the reduced shards exist only on the two-pass (clipping) path
            zeros = self._count_zeros(self._reduced)
        if need_clip:
            coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0).reshape(1).float()
            for i in range(len(self.shards)):
                launch(1, i, coef)
        arena.barrier(1)  # every rank has written its parameter shard into every peer
        self._shard_grads = [None] * len(self.shards)
        self.last_path = "fused"
        return True, norm, zeros

    @torch.no_grad()
    def step(self):
        if self._shard_grads[0] is None:
            self.reduce_gradients()
        if self.fused:
            return self._fused_step()
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        wd_base = self.param_groups[0]["weight_decay"]
        norm = self._global_grad_norm()
        zeros = self._count_zeros(self._shard_grads) if self.log_num_zeros else None
        coef = None
        if self.clip_grad and self.clip_grad > 0:
            coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0).reshape(1).float()
        for i, (s, e, wd) in enumerate(self.shards):
            p16 = self.buf.params[s:e]
            gsh = self._shard_grads[i]
            if gsh.dtype != torch.float32:
                gsh = gsh.float()
            ops.adamw_step(self.master[i], p16, self.exp_avg[i], self.exp_avg_sq[i], gsh, lr=lr,
                           beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                           wd=wd_base if wd else 0.0, step=self.step_count, grad_scale=self.grad_scale,
                           grad_scale_tensor=coef)
        if self.sharded:
            for (s, e, _), (rs, re, _) in zip(self.shards, self.buf.regions()):
                dist.all_gather_into_tensor(self.buf.params[rs:re], self.buf.params[s:e].clone(), group=self.group)
        self._shard_grads = [None] * len(self.shards)
        return True, norm, zeros

    def _count_zeros(self, shard_grads) -> torch.Tensor:
        """Number of exactly-zero elements of the reduced gradient (``--log-num-zeros-in-grad``); every element
        belongs to one shard, so the shard counts add up over the group."""
        n = sum((g == 0).sum() for g in shard_grads).to(torch.float32)
        if self.sharded and self.world > 1:
            dist.all_reduce(n, op=dist.ReduceOp.SUM, group=self.group)
        return n

    def zero_grad(self, set_to_none: bool = True):
        self.buf.zero_grads()
        self._shard_grads = [None] * len(self.shards)

    def get_loss_scale(self):
        return torch.ones((), device=self.buf.params.device)

    def reload_model_params(self):
        """Refresh fp32 master weights from the (bf16) model parameters, e.g. after loading a checkpoint."""
        for i, (s, e, _) in enumerate(self.shards):
            self.master[i].copy_(self.buf.params[s:e].float())

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        return dict(step=self.step_count, param_groups=self.param_groups, sharded=self.sharded,
                    world=self.world, shards=[(s, e) for s, e, _ in self.shards],
                    master=[t.cpu() for t in self.master], exp_avg=[t.cpu() for t in self.exp_avg],
                    exp_avg_sq=[t.cpu() for t in self.exp_avg_sq])

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.param_groups[0].update(sd["param_groups"][0])
        assert [tuple(x) for x in sd["shards"]] == [(s, e) for s, e, _ in self.shards], \
            "optimizer shard layout differs from the checkpoint"
        for dst, src in ((self.master, sd["master"]), (self.exp_avg, sd["exp_avg"]),
                         (self.exp_avg_sq, sd["exp_avg_sq"])):
            for d, s_ in zip(dst, src):
                d.copy_(s_)

    def gather_full_state(self, gloo_group=None):
        """Full-length fp32 (master, exp_avg, exp_avg_sq) on group rank 0 (None elsewhere): the
        ``distrib_optim.pt`` payload (teletron/train/checkpoint/checkpoint.py:72-76)."""
        if not self.sharded:
            full = {k: torch.cat([t.cpu() for t in v]) for k, v in
                    (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq))}
            return full
        out = {}
        for key, lst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            pieces = []
            for t in lst:
                gathered = [torch.empty_like(t) for _ in range(self.world)]
                dist.all_gather(gathered, t, group=self.group)
                pieces.append(torch.cat([x.cpu() for x in gathered]))
            out[key] = torch.cat(pieces)
        return out if self.rank == 0 else None

    def scatter_full_state(self, full):
        """Inverse of gather_full_state: every rank passes the full dict and keeps its slices."""
        pos = 0
        for i, ((s, e, _), (rs, re, _)) in enumerate(zip(self.shards, self.buf.regions())):
            for key, lst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                lst[i].copy_(full[key][pos + (s - rs): pos + (e - rs)])
            pos += re - rs


class DistributedDataParallel(torch.nn.Module):
    """The reference's DDP wrapper surface (teletron/core/distributed/distributed_data_parallel.py:40-298) over
    ``ParamBuffer``: ``forward``, ``no_sync()``, ``start_grad_sync()`` / ``finish_grad_sync()``,
    ``zero_grad_buffer()``, ``broadcast_params()``, ``scale_gradients()`` and the state-dict passthroughs, for code
    written against those names.  The trainer itself drives ``ParamBuffer`` + ``DistributedOptimizer`` directly.

    Gradients accumulate in the flat fp32 buffer over micro-batches; ``finish_grad_sync`` sums them over
    ``group`` and scales by ``1 / data_parallel_world_size``-style ``grad_scale`` (default ``1 / group size``).
    Inside ``no_sync()`` the sync calls do nothing, as in the reference."""

    def __init__(self, module: torch.nn.Module, group=None, grad_dtype=torch.float32, grad_scale: float = None,
                 broadcast: bool = True):
        super().__init__()
        self.module = module
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.buffer = ParamBuffer(module, shard_world=1, grad_dtype=grad_dtype)
        self.grad_scale = (1.0 / self.world) if grad_scale is None else float(grad_scale)
        self._sync_enabled = True
        self._pending = None
        if broadcast and self.world > 1:
            self.broadcast_params()

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        prev, self._sync_enabled = self._sync_enabled, False
        try:
            yield
        finally:
            self._sync_enabled = prev

    def start_grad_sync(self, *unused):
        """Fold autograd gradients into the flat buffer, scale, and launch the all-reduce asynchronously."""
        if not self._sync_enabled:
            return
        self.buffer.collect_grads()
        if self.grad_scale != 1.0:
            self.buffer.grads.mul_(self.grad_scale)
        if self.world > 1:
            self._pending = dist.all_reduce(self.buffer.grads, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def finish_grad_sync(self):
        if not self._sync_enabled:
            return
        if self._pending is None:
            self.start_grad_sync()
        if self._pending is not None:
            self._pending.wait()
            self._pending = None

    def scale_gradients(self, factor: float):
        self.buffer.grads.mul_(factor)

    def zero_grad_buffer(self):
        self.buffer.zero_grads()

    def broadcast_params(self):
        """Every rank takes the parameters of the first rank of the group."""
        if self.world > 1:
            src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
            dist.broadcast(self.buffer.params, src=src, group=self.group)

    def state_dict(self, prefix="", keep_vars=False):
        return self.module.state_dict(prefix=prefix, keep_vars=keep_vars)

    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        fn = getattr(self.module, "state_dict_for_save_checkpoint", None)
        return fn(prefix=prefix, keep_vars=keep_vars) if fn else self.state_dict(prefix, keep_vars)

    def load_state_dict(self, state_dict, strict=True):
        return self.module.load_state_dict(state_dict, strict=strict)
