"""Flat parameter / gradient buffers cut into buckets, data-parallel gradient reduction overlapped with
backward, and the (optionally sharded) AdamW optimizer with fp32 master weights.

What the reference spreads over its DDP wrapper, bucketed grad buffer and Megatron's
optimizers (teletron/core/distributed/distributed_data_parallel.py:14-298,
teletron/core/distributed/param_and_grad_buffer.py:31-520, teletron/train/lr_scheduler.py:423-509)
is two objects here:

  * ``ParamBuffer`` re-points every parameter into one contiguous bf16 buffer and gives it a
    ``main_grad`` view into one contiguous fp32 buffer.  Weight gradients are accumulated into
    ``main_grad`` by the wgrad GEMM epilogue; small parameters (biases, norms, modulation) get
    ordinary ``.grad`` tensors that are folded in by one multi-tensor kernel.  The buffer is laid out
    in up to four regions (weight decay or not, replicated across the tensor-parallel group or not);
    inside a region parameters sit in REVERSE definition order, as in the reference
    (param_and_grad_buffer.py:292), so that backward completes the region front to back, and the
    region is cut into uniform buckets (default 40 M elements, distributed_data_parallel.py:51).
    Every rank owns the same 1/world share of every bucket.
  * ``DistributedOptimizer`` reduces gradients over the DP x CP group bucket by bucket — a
    reduce-scatter straight on the fp32 buffer when sharded (the reference all-reduces through a
    400 MB fp32 staging copy, param_and_grad_buffer.py:128-148) — computes the global gradient
    norm, runs the fused AdamW kernel on the owned shares and all-gathers the bf16 parameters.
    With ``overlap`` a bucket's reduction is launched on a side stream as soon as the last
    micro-batch's backward has produced its last gradient (the contract of ``register_grad_ready``,
    param_and_grad_buffer.py:173-188); only the AdamW pass, which needs the global norm, waits for
    the end of backward.  The launches are the same with and without overlap, so the results are
    bit-identical.
  * gradient scale: all parameter gradients are partial sums over the CP group (the loss is
    normalised by the full token count), so the reduction is a plain sum and the scale is
    ``1 / dp`` (times ``1 / num_microbatches`` folded into the loss).
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..utils.nvtx import nvtx_range

_ALIGN = 8  # elements; keeps every parameter 16-byte aligned in the bf16 buffer
DEFAULT_BUCKET_ELEMS = 40_000_000


def _no_weight_decay(name: str, p: torch.Tensor) -> bool:
    """Megatron's default grouping: biases and 1-D parameters are not decayed."""
    return name.endswith(".bias") or p.dim() == 1


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class Region:
    """A contiguous range of the flat buffers whose elements share weight decay and tensor-parallel role,
    cut into ``n_buckets`` buckets of ``bucket_elems`` elements (the last one ``last_elems``)."""
    start: int
    end: int
    wd: bool
    tp_replicated: bool
    bucket_elems: int
    n_buckets: int = 1
    last_elems: int = 0

    def __post_init__(self):
        n = self.end - self.start
        self.n_buckets = max(1, (n + self.bucket_elems - 1) // self.bucket_elems)
        self.last_elems = n - (self.n_buckets - 1) * self.bucket_elems

    def __iter__(self):  # (start, end, wd) for code written against the two-region layout
        return iter((self.start, self.end, self.wd))

    def bucket_span(self, b: int) -> Tuple[int, int]:
        s = self.start + b * self.bucket_elems
        return s, min(s + self.bucket_elems, self.end)


@dataclass
class Bucket:
    gid: int
    region: int
    index: int
    start: int
    end: int
    params: List[str] = field(default_factory=list)


class ParamBuffer:
    def __init__(self, module: torch.nn.Module, shard_world: int = 1, grad_dtype=torch.float32, arena=None,
                 bucket_size: Optional[int] = None, tp_sharded_names: Optional[Iterable[str]] = None):
        """``arena``: a ``dist.SymmetricArena``; when given, both flat buffers live in symmetric peer
        memory so the fused reduce-scatter / AdamW / all-gather kernels can reach every rank's copy.
        ``bucket_size``: elements per bucket of the weight-decay regions (None: one bucket per region).
        ``tp_sharded_names``: under tensor parallelism, the parameters that hold a shard; every other
        parameter is replicated across the tensor-parallel group and goes to a region of its own."""
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        assert named, "module has no trainable parameters"
        dev = named[0][1].device
        self.param_dtype = named[0][1].dtype
        self.grad_dtype = grad_dtype
        self.shard_world = max(int(shard_world), 1)
        self.region_align = self.shard_world * 4 * _ALIGN
        sharded = None if tp_sharded_names is None else set(tp_sharded_names)
        groups: Dict[Tuple[bool, bool], List] = {(True, False): [], (True, True): [], (False, False): [], (False, True): []}
        for n, p in named:
            rep = sharded is not None and n not in sharded
            groups[(not _no_weight_decay(n, p), rep)].append((n, p))
        self.index: Dict[str, Tuple[int, int, torch.Size]] = {}
        self.regions_list: List[Region] = []
        off = 0
        for (wd, rep), members in groups.items():
            if not members:
                continue
            start = off
            for n, p in reversed(members):
                self.index[n] = (off, p.numel(), p.shape)
                off += _round_up(p.numel(), _ALIGN)
            off = _round_up(off, self.region_align)
            be = _round_up(int(bucket_size), self.region_align) if (bucket_size and wd) else off - start
            self.regions_list.append(Region(start, off, wd, rep, max(be, self.region_align)))
        self.numel = off
        self.decay_end = next((r.start for r in self.regions_list if not r.wd), self.numel)
        # buckets in firing order (region by region, front to back) and the buckets each parameter touches
        self.buckets: List[Bucket] = []
        for ri, r in enumerate(self.regions_list):
            for b in range(r.n_buckets):
                s, e = r.bucket_span(b)
                self.buckets.append(Bucket(len(self.buckets), ri, b, s, e))
        self.param_buckets: Dict[str, List[int]] = {}
        for n, (o, cnt, _) in self.index.items():
            hit = [bk.gid for bk in self.buckets if bk.start < o + cnt and o < bk.end]
            self.param_buckets[n] = hit
            for g in hit:
                self.buckets[g].params.append(n)
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
        self.by_name = dict(named)
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

    def collect_grads(self, names: Optional[Iterable[str]] = None):
        """Fold autograd ``.grad`` tensors (parameters not written by a wgrad epilogue) into main_grad:
        one multi-tensor kernel per 48 tensors on a GPU."""
        ps = [p for _, p in self.named] if names is None else [self.by_name[n] for n in names]
        ps = [p for p in ps if p.grad is not None]
        if not ps:
            return
        fast = [p for p in ps if p.grad.is_cuda and p.grad.dtype == torch.bfloat16 and p.grad.is_contiguous()
                and p.main_grad.dtype == torch.float32]
        if fast:
            from ..ops import _lib

            L = _lib.lib()
            cap = L.tt_multi_fold_max()
            for i in range(0, len(fast), cap):
                chunk = fast[i:i + cap]
                k = len(chunk)
                src = (_lib.c_ll * k)(*[p.grad.data_ptr() for p in chunk])
                dst = (_lib.c_ll * k)(*[p.main_grad.data_ptr() for p in chunk])
                cnt = (_lib.c_int * k)(*[p.grad.numel() for p in chunk])
                _lib.check(L.tt_multi_fold(src, dst, cnt, _lib.c_int(k), _lib.stream()), "tt_multi_fold")
        done = set(map(id, fast))
        for p in ps:
            if id(p) not in done:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
            p.grad = None

    def regions(self) -> List[Region]:
        return list(self.regions_list)


class DistributedOptimizer:
    """AdamW over a ParamBuffer. ``group``: the DP x CP process group (None = single process).

    ``sharded=True`` is the ZeRO-1 layout (``--use-distributed-optimizer``): each rank keeps fp32
    master / m / v for its 1/world share of every bucket ("owned-flat" order: the shares of a region's
    buckets one after the other).  ``grad_scale`` is applied to the summed gradient (use 1/dp).
    ``step()`` returns (ok, grad_norm, num_zeros) like Megatron's optimizers.

    ``overlap`` (``--overlap-grad-reduce``): call ``begin_last_microbatch()`` before the forward of the
    last micro-batch; its backward then launches each bucket's reduction when the bucket's last
    gradient is there (``param.grad_ready`` from the wgrad GEMM, a post-accumulate hook for the rest).
    Buckets start strictly in buffer order on every rank; what has not started by the end of backward
    starts in ``reduce_gradients()``.  A parameter is taken to receive ONE gradient per backward pass.
    """

    def __init__(self, buf: ParamBuffer, group=None, *, lr=1e-4, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.01, clip_grad=0.0, sharded=False, grad_scale=1.0, tp_group=None,
                 tp_sharded_names=(), overlap=False, comm_blocks: int = 0, kind: str = "adam", momentum: float = 0.9):
        """``tp_group``: under tensor parallelism the gradients of the regions that are replicated across
        the TP group are partial sums over that group's row shards and are all-reduced over it before the
        DP x CP reduction; the squared norm of the sharded regions is summed over it.  (The buffer must
        have been built with the same ``tp_sharded_names``.)"""
        assert kind in ("adam", "sgd"), kind
        self.kind, self.momentum = kind, momentum      # "sgd": momentum SGD (teletron/train/lr_scheduler.py:373-379)
        self.buf, self.group = buf, group
        self.tp_group = tp_group
        self.tp_world = dist.get_world_size(tp_group) if tp_group is not None else 1
        if tp_group is not None:
            assert any(r.tp_replicated for r in buf.regions_list) or not set(buf.index) - set(tp_sharded_names), \
                "under tensor parallelism build the ParamBuffer with tp_sharded_names"
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.sharded = bool(sharded) and self.world > 1
        self.sw = self.world if self.sharded else 1           # ranks that split a bucket
        assert buf.region_align % (self.sw * 4) == 0, "ParamBuffer was built for a smaller shard_world"
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.clip_grad, self.grad_scale = clip_grad, grad_scale
        self.step_count = 0
        self.param_groups = [dict(lr=lr, weight_decay=weight_decay)]  # scheduler-facing view
        self.regions = buf.regions()
        self.shards: List[Tuple[int, int, bool]] = [(r.start, r.end, r.wd) for r in self.regions] if not self.sharded \
            else [(-1, -1, r.wd) for r in self.regions]        # contiguous only when nothing is sharded
        dev = buf.params.device
        self.master = [self._owned(buf.params, r).float().clone() for r in self.regions]
        self.exp_avg = [torch.zeros_like(t) for t in self.master]
        self.exp_avg_sq = [torch.zeros_like(t) for t in self.master]
        self._shard_grads: List[Optional[torch.Tensor]] = [None] * len(self.regions)
        self._reduced: Optional[List[torch.Tensor]] = None
        self._p16: Optional[List[torch.Tensor]] = None
        # fused path: peer-memory reduce-scatter + AdamW + parameter scatter (csrc/comm.cu)
        self.fused = bool(self.sharded and buf.arena is not None and buf.grads.dtype == torch.float32
                          and kind == "adam")
        self.overlap = bool(overlap) and self.world > 1
        self.comm_blocks = int(comm_blocks)
        self.log_num_zeros = False
        self.last_path = "nccl"
        self.fired_in_backward = 0       # buckets whose reduction started before backward ended (last step)
        # per-step bucket state
        nb = len(buf.buckets)
        self._fired = [False] * nb
        self._next = 0
        self._armed = False
        self._pending_params: List[int] = [0] * nb
        self._param_seen: Dict[str, bool] = {}
        self._handles: list = []
        self._tp_reduced = False
        self._side = None
        self._barrier_done = False
        if self.fused:
            from ..ops import _lib

            self._blocks = self.comm_blocks or _lib.lib().tt_comm_blocks()
            self._partials = torch.zeros((nb, self._blocks), dtype=torch.float32, device=dev)
            self._ss_slots = buf.arena.alloc(buf.arena.max_peers, torch.float32)
            self._ss_slots.tensor.zero_()
            self._norm_out = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.overlap:
            self._install_hooks()

    # ------------------------------------------------------------------ owned-flat <-> global
    def _share(self, r: Region, b: int) -> int:
        return (r.last_elems if b == r.n_buckets - 1 else r.bucket_elems) // self.sw

    def _owned_spans(self, r: Region, rank: Optional[int] = None):
        """(flat_start, global_start, length) of each bucket's share owned by ``rank``."""
        rank = self.rank if rank is None else rank
        full = r.bucket_elems // self.sw
        for b in range(r.n_buckets):
            n = self._share(r, b)
            yield b * full, r.start + b * r.bucket_elems + (rank if self.sharded else 0) * n, n

    def _owned(self, flat: torch.Tensor, r: Region, rank: Optional[int] = None) -> torch.Tensor:
        """The elements of a full-length buffer that ``rank`` owns in region ``r``, in owned-flat order."""
        if not self.sharded:
            return flat[r.start:r.end]
        return torch.cat([flat[g:g + n] for _, g, n in self._owned_spans(r, rank)])

    def owned_len(self, r: Region) -> int:
        return (r.end - r.start) // self.sw

    # ------------------------------------------------------------------ gradient-ready bookkeeping
    def _install_hooks(self):
        for n, p in self.buf.named:
            p.grad_ready = (lambda name=n: self._param_ready(name))
            # autograd runs this hook for every parameter of the graph, also with an undefined gradient when the
            # wgrad GEMM has already accumulated into main_grad (and reported through grad_ready)
            p.register_post_accumulate_grad_hook(lambda _p, name=n: self._param_ready(name, _p.grad is not None))

    def begin_last_microbatch(self):
        """Arm the gradient-ready hooks: from here on a bucket's reduction starts as soon as every parameter in
        it has received its gradient."""
        if not self.overlap:
            return
        self._armed = True
        self._param_seen = {}
        for bk in self.buf.buckets:
            self._pending_params[bk.gid] = len(bk.params)

    def _param_ready(self, name: str, has_grad: bool = True):
        if not self._armed:
            return
        if self._param_seen.get(name):
            if has_grad and any(self._fired[g] for g in self.buf.param_buckets[name]):
                raise RuntimeError(f"{name} received another gradient after its bucket's reduction had started; "
                                   "parameters used more than once per backward need --no-overlap-grad-reduce")
            return
        self._param_seen[name] = True
        for g in self.buf.param_buckets[name]:
            self._pending_params[g] -= 1
        self._fire_ready()

    def _fire_ready(self, force: bool = False):
        """Start reductions in buffer order: bucket k only after bucket k-1, so that every rank issues the same
        sequence of collectives / peer barriers."""
        nb = len(self.buf.buckets)
        while self._next < nb:
            bk = self.buf.buckets[self._next]
            r = self.regions[bk.region]
            if not force:
                if self._pending_params[bk.gid] > 0:
                    return
                if r.tp_replicated and self.tp_group is not None:
                    return          # needs the tensor-parallel all-reduce first: done in reduce_gradients()
            self._fire(bk, in_backward=not force)
            self._next += 1

    def _fire(self, bk: Bucket, in_backward: bool):
        self.buf.collect_grads(bk.params)
        self._fired[bk.gid] = True
        if in_backward:
            self.fired_in_backward += 1
        if self.world == 1:
            return
        if self.fused:
            self._fire_fused(bk, in_backward)
        else:
            self._fire_nccl(bk)

    def _fire_nccl(self, bk: Bucket):
        g = self.buf.grads
        r = self.regions[bk.region]
        seg = g[bk.start:bk.end]
        if not self.sharded:
            self._handles.append(dist.all_reduce(seg, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            return
        if self._reduced is None:
            self._reduced = [torch.empty(self.owned_len(x), dtype=torch.float32, device=g.device) for x in self.regions]
        n = self._share(r, bk.index)
        f0 = bk.index * (r.bucket_elems // self.sw)
        out = self._reduced[bk.region][f0:f0 + n]
        if g.is_cuda:
            self._handles.append(dist.reduce_scatter_tensor(out, seg, op=dist.ReduceOp.SUM, group=self.group,
                                                            async_op=True))
        else:  # gloo has no reduce-scatter: all-reduce the bucket and keep our share
            dist.all_reduce(seg, op=dist.ReduceOp.SUM, group=self.group)
            out.copy_(seg[self.rank * n:(self.rank + 1) * n])

    def _fire_fused(self, bk: Bucket, in_backward: bool):
        """Pass 1 of K-DP-RS-ADAMW for one bucket: peer barrier, then pull-reduce of the owned share from every
        peer.  During backward both run on a side stream behind an event of the compute stream."""
        from ..ops import _lib

        buf, arena, r = self.buf, self.buf.arena, self.regions[bk.region]
        cur = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream()
        if in_backward:
            self._side.wait_stream(cur)
            stream_ctx = torch.cuda.stream(self._side)
        else:
            if self._side_used:
                cur.wait_stream(self._side)      # keep bucket order: the side stream's buckets come first
                self._side_used = False
            stream_ctx = contextlib.nullcontext()
        with stream_ctx, nvtx_range(f"dp_reduce_bucket_{bk.gid}"):
            if self.overlap or not self._barrier_done:
                # every rank's gradients of this bucket (and of all earlier ones) are complete; with overlap one
                # barrier per bucket, whichever stream it runs on, so that every rank issues the same sequence
                arena.barrier(2)
                self._barrier_done = True
            rc = _lib.lib().tt_dp_bucket_step(
                _lib.c_int(0), buf.symm_grads.c_ptrs(), buf.symm_params.c_ptrs(), _lib.c_int(self.world),
                _lib.c_int(self.rank), _lib.c_ll(r.start), _lib.c_ll(r.bucket_elems), _lib.c_ll(r.last_elems),
                _lib.c_int(r.n_buckets), _lib.c_int(bk.index), _lib.c_int(bk.index + 1),
                None, None, None, None, _lib.c_float(self.grad_scale), None, None,
                _lib.c_float(0.0), None, _lib.c_float(0.0), _lib.c_float(0.0), _lib.c_float(0.0), _lib.c_float(0.0),
                _lib.c_float(0.0), _lib.c_int(1), _lib.ptr(self._partials[bk.gid]), _lib.c_int(self._blocks),
                _lib.stream())
            _lib.check(rc, "tt_dp_bucket_step")
        if in_backward:
            self._side_used = True

    _side_used = False

    # ------------------------------------------------------------------ gradient sync
    def reduce_gradients(self):
        """Finish the reduction over the group; afterwards ``_shard_grads`` holds this rank's fp32 shares."""
        self._armed = False
        g = self.buf.grads
        self.buf.collect_grads()       # whatever autograd left in .grad, in one multi-tensor pass
        if self.tp_group is not None and not self._tp_reduced:
            for r in self.regions:
                if r.tp_replicated:
                    dist.all_reduce(g[r.start:r.end], op=dist.ReduceOp.SUM, group=self.tp_group)
            self._tp_reduced = True
        self._fire_ready(force=True)
        for h in self._handles:
            if h is not None:
                h.wait()
        self._handles = []
        if self.fused and self._side_used:
            torch.cuda.current_stream().wait_stream(self._side)
            self._side_used = False
        if self.fused:
            self._shard_grads = ["in place"] * len(self.regions)    # each share's sum sits in this rank's gradient buffer
        elif self.world > 1 and self.sharded:
            self._shard_grads = list(self._reduced)
        else:
            self._shard_grads = [g[r.start:r.end] for r in self.regions]

    def _sum_of_squares(self) -> torch.Tensor:
        """Squared L2 norm of the whole (unscaled) reduced gradient, identical on every rank of the DP x CP x TP
        grid: sharded regions add up over the tensor-parallel group, replicated regions count once."""
        ss_sh = ss_rep = None
        for r, gsh in zip(self.regions, self._shard_grads):
            t = ops.grad_norm(gsh.float() if gsh.dtype != torch.float32 else gsh)[2]
            if r.tp_replicated:
                ss_rep = t if ss_rep is None else ss_rep + t
            else:
                ss_sh = t if ss_sh is None else ss_sh + t
        return self._combine_ss(ss_sh, ss_rep)

    def _combine_ss(self, ss_sh, ss_rep):
        zero = None
        for t in (ss_sh, ss_rep):
            if t is not None:
                zero = torch.zeros_like(t)
        ss_sh = zero if ss_sh is None else ss_sh
        ss_rep = zero if ss_rep is None else ss_rep
        if self.sharded:       # each rank holds 1/world of both kinds
            both = torch.stack([ss_sh.reshape(()), ss_rep.reshape(())])
            dist.all_reduce(both, op=dist.ReduceOp.SUM, group=self.group)
            ss_sh, ss_rep = both[0], both[1]
        if self.tp_group is not None:
            ss_sh = ss_sh.clone()
            dist.all_reduce(ss_sh, op=dist.ReduceOp.SUM, group=self.tp_group)
        return ss_sh + ss_rep

    def _global_grad_norm(self) -> torch.Tensor:
        return self._sum_of_squares().sqrt() * self.grad_scale

    # ------------------------------------------------------------------ step
    def _bucket_step(self, mode, ri, coef, ss_slots, b0=0, b1=None, partial=None):
        from ..ops import _lib

        buf, r = self.buf, self.regions[ri]
        lr = self.param_groups[0]["lr"]
        wd = self.param_groups[0]["weight_decay"] if r.wd else 0.0
        rc = _lib.lib().tt_dp_bucket_step(
            _lib.c_int(mode), buf.symm_grads.c_ptrs(), buf.symm_params.c_ptrs(), _lib.c_int(self.world),
            _lib.c_int(self.rank), _lib.c_ll(r.start), _lib.c_ll(r.bucket_elems), _lib.c_ll(r.last_elems),
            _lib.c_int(r.n_buckets), _lib.c_int(b0), _lib.c_int(r.n_buckets if b1 is None else b1),
            None, _lib.ptr(self.master[ri]),
            _lib.ptr(self.exp_avg[ri]), _lib.ptr(self.exp_avg_sq[ri]), _lib.c_float(self.grad_scale),
            _lib.ptr(coef), _lib.ptr(ss_slots), _lib.c_float(self.clip_grad or 0.0),
            _lib.ptr(self._norm_out if ss_slots is not None else None), _lib.c_float(lr),
            _lib.c_float(self.betas[0]), _lib.c_float(self.betas[1]), _lib.c_float(self.eps), _lib.c_float(wd),
            _lib.c_int(self.step_count), _lib.ptr(partial), _lib.c_int(0), _lib.stream())
        _lib.check(rc, "tt_dp_bucket_step")

    @torch.no_grad()
    def _fused_step(self):
        """K-DP-RS-ADAMW, pass 2: every rank's share of the squared norm is exchanged through peer memory, then one
        kernel per region clips, runs AdamW on the owned shares and stores the new bf16 parameters into every
        peer; a barrier closes the step.  (Pass 1, the pull-reduce per bucket, ran in ``reduce_gradients`` or,
        with overlap, during backward.)"""
        from ..ops import _lib

        L = _lib.lib()
        buf, arena = self.buf, self.buf.arena
        self.step_count += 1
        with nvtx_range("dp_adamw_scatter"):
            return self._fused_step_body(L, arena)

    def _fused_step_body(self, L, arena):
        from ..ops import _lib

        buf = self.buf
        zeros = None
        if self.log_num_zeros:
            zeros = self._count_zeros([self._owned(buf.grads, r) for r in self.regions])
        if self.tp_group is None:
            rc = L.tt_dp_norm_exchange(_lib.ptr(self._partials), _lib.c_int(self._partials.numel()),
                                       self._ss_slots.c_ptrs(), _lib.c_int(self.world), _lib.c_int(self.rank),
                                       _lib.stream())
            _lib.check(rc, "tt_dp_norm_exchange")
            arena.barrier(0)      # every rank's share of the norm has landed; every rank's backward is complete
            for ri in range(len(self.regions)):
                self._bucket_step(1, ri, None, self._ss_slots.tensor)
            norm = self._norm_out.clone().reshape(())
        else:
            nb = 0
            ss_sh = ss_rep = None
            for r in self.regions:      # bucket rows of the partial sums, region by region
                t = self._partials[nb:nb + r.n_buckets].sum()
                nb += r.n_buckets
                if r.tp_replicated:
                    ss_rep = t if ss_rep is None else ss_rep + t
                else:
                    ss_sh = t if ss_sh is None else ss_sh + t
            norm = self._combine_ss(ss_sh, ss_rep).sqrt() * self.grad_scale
            coef = None
            if self.clip_grad and self.clip_grad > 0:
                coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0).reshape(1).float()
            arena.barrier(0)
            for ri in range(len(self.regions)):
                self._bucket_step(1, ri, coef, None)
        arena.barrier(1)  # every rank has written its parameter shares into every peer
        self.last_path = "fused"
        return True, norm, zeros

    @torch.no_grad()
    def step(self):
        if self._shard_grads[0] is None:
            self.reduce_gradients()
        try:
            if self.fused:
                return self._fused_step()
            return self._plain_step()
        finally:
            self._end_of_step()

    def _end_of_step(self):
        nb = len(self.buf.buckets)
        self._shard_grads = [None] * len(self.regions)
        self._fired = [False] * nb
        self._next = 0
        self._tp_reduced = False
        self._barrier_done = False
        self._armed = False

    def _plain_step(self):
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        wd_base = self.param_groups[0]["weight_decay"]
        norm = self._global_grad_norm()
        zeros = self._count_zeros(self._shard_grads) if self.log_num_zeros else None
        coef = None
        if self.clip_grad and self.clip_grad > 0:
            coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0).reshape(1).float()
        if self.sharded and self._p16 is None:
            self._p16 = [torch.empty(self.owned_len(r), dtype=self.buf.params.dtype, device=self.buf.params.device)
                         for r in self.regions]
        for i, r in enumerate(self.regions):
            p16 = self._p16[i] if self.sharded else self.buf.params[r.start:r.end]
            gsh = self._shard_grads[i]
            if gsh.dtype != torch.float32:
                gsh = gsh.float()
            if self.kind == "sgd":     # exp_avg is the momentum buffer; weight decay added to the gradient
                g32 = gsh * (self.grad_scale if coef is None else self.grad_scale * coef)
                if r.wd and wd_base:
                    g32 = g32.add(self.master[i], alpha=wd_base)
                self.exp_avg[i].mul_(self.momentum).add_(g32)
                self.master[i].add_(self.exp_avg[i], alpha=-lr)
                p16.copy_(self.master[i])
                continue
            ops.adamw_step(self.master[i], p16, self.exp_avg[i], self.exp_avg_sq[i], gsh, lr=lr,
                           beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                           wd=wd_base if r.wd else 0.0, step=self.step_count, grad_scale=self.grad_scale,
                           grad_scale_tensor=coef)
        if self.sharded:
            handles = []
            for i, r in enumerate(self.regions):
                for b in range(r.n_buckets):
                    s, e = r.bucket_span(b)
                    f0, n = b * (r.bucket_elems // self.sw), self._share(r, b)
                    handles.append(dist.all_gather_into_tensor(self.buf.params[s:e], self._p16[i][f0:f0 + n],
                                                               group=self.group, async_op=True))
            for h in handles:
                h.wait()
        return True, norm, zeros

    def _count_zeros(self, shard_grads) -> torch.Tensor:
        """Number of exactly-zero elements of the reduced gradient (``--log-num-zeros-in-grad``); every element
        belongs to one share, so the counts add up over the group."""
        n = sum((g == 0).sum() for g in shard_grads).to(torch.float32)
        if self.sharded and self.world > 1:
            dist.all_reduce(n, op=dist.ReduceOp.SUM, group=self.group)
        return n

    def zero_grad(self, set_to_none: bool = True):
        self.buf.zero_grads()
        self._shard_grads = [None] * len(self.regions)
        self.fired_in_backward = 0

    def get_loss_scale(self):
        return torch.ones((), device=self.buf.params.device)

    def reload_model_params(self):
        """Refresh fp32 master weights from the (bf16) model parameters, e.g. after loading a checkpoint."""
        for i, r in enumerate(self.regions):
            self.master[i].copy_(self._owned(self.buf.params, r).float())

    # ------------------------------------------------------------------ checkpoint
    def layout(self) -> dict:
        """What a reader needs to place the flat optimizer state: parameter offsets and region / bucket geometry."""
        return dict(numel=self.buf.numel, world=self.sw,
                    index={k: (o, n) for k, (o, n, _) in self.buf.index.items()},
                    regions=[(r.start, r.end, r.wd, r.tp_replicated, r.bucket_elems) for r in self.regions])

    def state_dict(self):
        return dict(step=self.step_count, param_groups=self.param_groups, sharded=self.sharded,
                    world=self.world, layout=self.layout(),
                    master=[t.cpu() for t in self.master], exp_avg=[t.cpu() for t in self.exp_avg],
                    exp_avg_sq=[t.cpu() for t in self.exp_avg_sq])

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.param_groups[0].update(sd["param_groups"][0])
        lay = sd.get("layout")
        if lay is not None and (lay["index"] != self.layout()["index"] or lay["world"] != self.sw):
            raise RuntimeError("optimizer buffer layout differs from the checkpoint (different model, tensor-parallel "
                               "size or sharding); load through distrib_optim.pt or use --no-load-optim")
        for dst, src in ((self.master, sd["master"]), (self.exp_avg, sd["exp_avg"]),
                         (self.exp_avg_sq, sd["exp_avg_sq"])):
            assert len(dst) == len(src), "optimizer region count differs from the checkpoint"
            for d, s_ in zip(dst, src):
                d.copy_(s_)

    def gather_full_state(self, gloo_group=None):
        """Full-length fp32 (master, exp_avg, exp_avg_sq) in buffer order plus the layout, on group rank 0
        (None elsewhere): the ``distrib_optim.pt`` payload (teletron/train/checkpoint/checkpoint.py:72-76).
        Collective: every rank of the group calls it.  The shares travel bucket by bucket to rank 0 only (one
        ``gather`` per bucket and state tensor), so the device holds one bucket's worth of staging at a time: a
        whole-state all-gather needs world x 15 GiB on every GPU of a 16 B-parameter model at four ranks."""
        out = {}
        root = dist.get_global_rank(self.group, 0) if (self.sharded and self.group is not None) else 0
        for key, lst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            full = torch.zeros(self.buf.numel, dtype=torch.float32) if self.rank == 0 else None
            for r, t in zip(self.regions, lst):
                if not self.sharded:
                    if full is not None:
                        full[r.start:r.end] = t.cpu()
                    continue
                spans = [list(self._owned_spans(r, rk)) for rk in range(self.world)]
                for bi, (f0, _, n) in enumerate(spans[self.rank]):
                    piece = t[f0:f0 + n].contiguous()
                    bufs = [torch.empty_like(piece) for _ in range(self.world)] if self.rank == 0 else None
                    dist.gather(piece, bufs, dst=root, group=self.group)
                    if self.rank == 0:
                        for rk, got in enumerate(bufs):
                            _, g0, nn = spans[rk][bi]
                            full[g0:g0 + nn] = got.cpu()
            out[key] = full
        out["layout"] = self.layout()
        return out if self.rank == 0 else None

    def scatter_full_state(self, full):
        """Inverse of gather_full_state: every rank passes the full dict and keeps its shares.  A state written
        under another layout (other DP x CP size, bucket size or parameter order) is re-placed parameter by
        parameter through the offsets stored with it."""
        lay = full.get("layout")
        mine = self.layout()
        same = lay is None or (lay["index"] == mine["index"] and lay["numel"] == mine["numel"])
        for key, lst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            src = full[key]
            if not same:
                if set(lay["index"]) != set(mine["index"]):
                    raise RuntimeError("distrib_optim.pt holds other parameters than this model")
                re = torch.zeros(self.buf.numel, dtype=torch.float32)
                for k, (o, n) in mine["index"].items():
                    so, sn = lay["index"][k]
                    if sn != n:
                        raise RuntimeError(f"distrib_optim.pt: {k} has {sn} elements, the model has {n} "
                                           "(different tensor-parallel size?)")
                    re[o:o + n] = src[so:so + n]
                src = re
            elif src.numel() != self.buf.numel:
                raise RuntimeError("distrib_optim.pt carries no layout and its length differs from this run's buffer")
            for i, r in enumerate(self.regions):
                lst[i].copy_(self._owned(src, r))


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
