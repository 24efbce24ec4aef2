"""Small public helpers that user scripts written against the reference import from its training utilities
(teletron/train/utils.py:40-54,195-312,594-612 and teletron/utils/aux_func.py:803-900): rank-filtered printing,
parameter / gradient norms, sample counts, iteration count under a batch-size ramp, memory reports.
"""
from __future__ import annotations

import time
from typing import Tuple

import torch
import torch.distributed as dist

from ..utils.flops import memory_report, theoretical_memory_gb, wan_flops_per_sample
from .microbatches import BatchSchedule


def _rank_world() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def is_last_rank() -> bool:
    r, w = _rank_world()
    return r == w - 1


def print_rank_0(message) -> None:
    if _rank_world()[0] == 0:
        print(message, flush=True)


def print_rank_last(message) -> None:
    if is_last_rank():
        print(message, flush=True)


def print_datetime(string: str) -> None:
    """Barrier, then rank 0 prints ``[string] datetime: ...`` (start-up and shutdown markers)."""
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    print_rank_0(f"[{string}] datetime: {time.strftime('%Y-%m-%d %H:%M:%S')} ")


def get_attr_wrapped_model(model, attr: str, allow_none: bool = True):
    """Attribute ``attr`` of the innermost module under ``.module`` wrappers (Float16Module and the like)."""
    while not hasattr(model, attr):
        if not hasattr(model, "module"):
            if allow_none:
                return None
            raise AttributeError(f"no wrapped module has an attribute {attr!r}")
        model = model.module
    return getattr(model, attr)


def calc_params_l2_norm(model) -> float:
    """L2 norm over all parameters of ``model`` (or a list of models), computed in fp32; parameters sharded by
    tensor parallelism (attribute ``tp_shard_dim``) are summed over the TP group, replicated ones counted once."""
    from ..parallel import state as mpu

    models = model if isinstance(model, (list, tuple)) else [model]
    tp = mpu.get_tensor_model_parallel_world_size() if mpu.model_parallel_is_initialized() else 1
    local = torch.zeros((), dtype=torch.float64)
    shared = torch.zeros((), dtype=torch.float64)
    for m in models:
        for p in m.parameters():
            ss = p.detach().double().pow(2).sum().cpu()
            if tp > 1 and getattr(p, "tp_shard_dim", None) is not None:
                local += ss
            else:
                shared += ss
    if tp > 1:
        t = local.to("cuda" if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(t, group=mpu.get_tensor_model_parallel_group())
        local = t.cpu()
    return float((local + shared).sqrt())


def get_grad_norm(model) -> float:
    """L2 norm of the ``.grad`` (or ``.main_grad``) tensors that exist, as the reference's fallback computes it."""
    ss = 0.0
    for p in model.parameters():
        g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
        if g is not None:
            ss += float(g.detach().double().pow(2).sum())
    return ss ** 0.5


def get_train_valid_test_num_samples(args) -> Tuple[int, int, int]:
    train = args.train_samples if getattr(args, "train_samples", None) else args.train_iters * args.global_batch_size
    eval_iters = (args.train_iters // max(args.eval_interval, 1) + 1) * args.eval_iters
    return train, eval_iters * args.global_batch_size, args.eval_iters * args.global_batch_size


def update_train_iters(args) -> int:
    """For sample-based training (``--train-samples``) derive ``args.train_iters``; under ``--rampup-batch-size``
    the ramp's smaller batches are stepped through first and a partial last batch is dropped."""
    if getattr(args, "train_iters", None):
        return args.train_iters
    if not getattr(args, "rampup_batch_size", None):
        args.train_iters = args.train_samples // args.global_batch_size
        return args.train_iters
    sched = BatchSchedule(args.global_batch_size, args.micro_batch_size, args.data_parallel_size, args.rampup_batch_size)
    iterations, consumed = 0, 0
    while consumed <= sched.ramp_samples:
        consumed += sched.global_batch_at(consumed)
        iterations += 1
    iterations += max(args.train_samples - consumed, 0) // args.global_batch_size
    args.train_iters = iterations
    return iterations


def report_memory(name: str) -> None:
    print(memory_report(f"[Rank {_rank_world()[0]}] {name}"), flush=True)


def report_theoretical_memory(args, num_params: int, verbose: bool = False) -> float:
    world = getattr(args, "data_parallel_size", 1) * getattr(args, "context_parallel_size", 1)
    gb = theoretical_memory_gb(num_params, world, bool(getattr(args, "use_distributed_optimizer", False)))
    print_rank_0(f"Theoretical memory footprint of weights, gradients and optimizer state: {gb:.2f} GiB per GPU")
    return gb


def num_floating_point_operations(cfg, tokens_per_sample: int, batch_size: int, recompute: bool = False) -> float:
    """Training FLOPs of ``batch_size`` samples of ``tokens_per_sample`` video tokens for a Wan configuration."""
    return wan_flops_per_sample(cfg, tokens_per_sample, recompute=recompute) * batch_size
