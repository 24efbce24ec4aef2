"""Checkpoint save / load in the Megatron directory layout the reference uses
(teletron/train/checkpoint/utils.py:47-113, teletron/train/checkpoint/checkpoint.py:46-398):

    <save>/latest_checkpointed_iteration.txt            integer iteration or "release"
    <save>/iter_0000100/mp_rank_00/model_optim_rng.pt   one directory per tensor-parallel rank
    <save>/iter_0000100/mp_rank_00/distrib_optim.pt     fp32 optimizer state when it is sharded

With ``--use-dist-ckpt`` the iteration directory holds a distributed checkpoint instead (the reference hands this
case to Megatron's ``dist_checkpointing.save(state_dict, dir, (format, 1))``, checkpoint.py:61-106,154-179):
``metadata.json`` (``sharded_backend`` = ``--dist-ckpt-format``), ``common.pt`` (everything that is not a tensor)
and the tensors written by every rank in parallel through ``torch.distributed.checkpoint`` — replicated model
tensors once (spread over the ranks with ``--ckpt-fully-parallel-save``), tensor-parallel shards and each rank's
share of the optimizer state under rank-qualified keys, so nothing is gathered to one rank.  On load the format is
taken from the flag or, with ``--auto-detect-ckpt-format``, from the presence of ``metadata.json``.

``model_optim_rng.pt`` is a ``torch.save`` dict with the keys ``args`` (argparse.Namespace),
``checkpoint_version`` (3.0), ``iteration``, ``model`` (bare parameter names such as
``blocks.0.self_attn.q.weight``, bf16), ``optimizer``, ``opt_param_scheduler``, ``rng_state`` and
``num_floating_point_operations_so_far``.  The file is written by data-parallel rank 0 of each
tensor-parallel rank through a temporary file and ``os.replace``; rank 0 updates the tracker
after a barrier.  Loading honours ``--finetune``, ``--no-load-optim``, ``--no-load-rng``,
``--ckpt-step``, ``--pretrained-checkpoint`` and ``--exit-on-missing-checkpoint``.
"""
from __future__ import annotations

import os
import random
import sys
from argparse import Namespace
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import state as mpu

TRACKER = "latest_checkpointed_iteration.txt"
MODEL_FILE = "model_optim_rng.pt"
DISTOPT_FILE = "distrib_optim.pt"


# ----------------------------------------------------------------------------- naming
def checkpoint_dir(root: str, iteration, release: bool = False) -> str:
    return os.path.join(root, "release" if release else f"iter_{int(iteration):07d}")


def checkpoint_name(root: str, iteration, release=False, tp_rank: Optional[int] = None,
                    pp_rank: Optional[int] = None, pp_size: int = 1, filename: str = MODEL_FILE) -> str:
    tp_rank = mpu.get_tensor_model_parallel_rank() if tp_rank is None else tp_rank
    sub = f"mp_rank_{tp_rank:02d}"
    if pp_size > 1:
        sub += f"_{(pp_rank or 0):03d}"
    return os.path.join(checkpoint_dir(root, iteration, release), sub, filename)


def _load_mapped(path: str):
    """``torch.load`` of a file every rank opens but reads only a part of (the gathered optimizer state: 12 bytes
    per parameter): memory-mapped, so a rank pages in its own shares instead of holding a private copy of the
    whole file; plain loading for files written in the legacy (non-zip) format."""
    try:
        return torch.load(path, map_location="cpu", weights_only=False, mmap=True)
    except (RuntimeError, ValueError):
        return torch.load(path, map_location="cpu", weights_only=False)


def zero2_shard_name(root: str, iteration, release: bool = False) -> str:
    """``zero2_optim_dp{d}_cp{c}.pt`` of this rank, beside its tensor-parallel rank's model file."""
    return checkpoint_name(root, iteration, release,
                           filename=f"zero2_optim_dp{mpu.get_data_parallel_rank()}_cp{mpu.get_context_parallel_rank()}.pt")


def tracker_filename(root: str) -> str:
    return os.path.join(root, TRACKER)


def read_tracker(root: str) -> Tuple[int, bool]:
    """(iteration, release). Raises FileNotFoundError when there is no tracker."""
    with open(tracker_filename(root)) as f:
        txt = f.read().strip()
    if txt == "release":
        return 0, True
    try:
        it = int(txt)
    except ValueError as e:
        raise ValueError(f"invalid tracker content {txt!r} in {tracker_filename(root)}") from e
    if dist.is_initialized() and dist.get_world_size() > 1:
        grp = mpu.get_transformer_model_group()
        dev = "cuda" if (torch.cuda.is_available() and dist.get_backend(grp) == "nccl") else "cpu"
        t = torch.tensor([it], dtype=torch.long, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=grp)
        it = int(t.item())
    return it, False


# ----------------------------------------------------------------------------- rng
def get_rng_state(per_dp_rank: bool = False):
    """``[state]`` of this rank, or, with ``per_dp_rank`` (``--data-parallel-random-init``: every data-parallel rank
    runs its own random stream), the states of all data-parallel ranks in rank order.  Collective in that case:
    every rank of the DP x CP group calls it."""
    st = dict(random_rng_state=random.getstate(), np_rng_state=np.random.get_state(),
              torch_rng_state=torch.get_rng_state(),
              cuda_rng_state=torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
              rng_tracker_states={})
    if per_dp_rank and dist.is_initialized() and mpu.model_parallel_is_initialized() \
            and mpu.get_data_parallel_world_size(with_context_parallel=True) > 1:
        grp = mpu.get_data_parallel_group(with_context_parallel=True)
        states = [None] * dist.get_world_size(grp)
        dist.all_gather_object(states, st, group=grp)
        return states
    return [st]


def set_rng_state(states, dp_rank: int = 0):
    st = states[dp_rank] if len(states) > dp_rank else states[0]
    random.setstate(st["random_rng_state"])
    np.random.set_state(st["np_rng_state"])
    torch.set_rng_state(st["torch_rng_state"])
    if st.get("cuda_rng_state") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda_rng_state"])


def _rng_index(args) -> int:
    """Which saved state this rank takes: its own when the run keeps one stream per data-parallel rank."""
    if getattr(args, "data_parallel_random_init", False) and mpu.model_parallel_is_initialized():
        return mpu.get_data_parallel_rank(with_context_parallel=True)
    return 0


def _atomic_save(obj, path: str):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _barrier():
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier(group=mpu.get_transformer_model_group())


def _plain_namespace(args) -> Namespace:
    keep = {}
    for k, v in vars(args).items():
        if isinstance(v, (int, float, str, bool, type(None), list, tuple, dict)) and k != "deferred_rng_state":
            keep[k] = v
    return Namespace(**keep)


# ----------------------------------------------------------------------------- distributed format
DIST_META = "metadata.json"
DIST_COMMON = "common.pt"


def is_dist_checkpoint(root: str, iteration, release: bool = False) -> bool:
    return os.path.exists(os.path.join(checkpoint_dir(root, iteration, release), DIST_META))


def _dist_tensor_dict(model, optimizer, args, with_optim: bool):
    """The tensors this rank contributes / expects, keyed so that equal keys mean equal (replicated) tensors:
    tensor-parallel shards carry the TP rank in their key, optimizer shares the rank in the DP x CP group too."""
    from ..parallel.tp import tp_shard_dims

    inner = model.module if hasattr(model, "module") else model
    tp_size = mpu.get_tensor_model_parallel_world_size()
    tp_rank = mpu.get_tensor_model_parallel_rank()
    sharded = set(tp_shard_dims(inner)) if tp_size > 1 else set()
    out = {}
    for k, v in inner.state_dict().items():
        key = f"model.{k}" + (f"@tp{tp_rank}of{tp_size}" if k in sharded else "")
        out[key] = v.detach()
    if with_optim and optimizer is not None:
        r = optimizer.rank if optimizer.sharded else 0
        w = optimizer.world if optimizer.sharded else 1
        for kind in ("master", "exp_avg", "exp_avg_sq"):
            for i, t in enumerate(getattr(optimizer, kind)):
                out[f"optimizer.{kind}.region{i}@tp{tp_rank}of{tp_size}@dp{r}of{w}"] = t
    return out


def _save_dist(iteration, model, optimizer, opt_param_scheduler, args, flops) -> str:
    import json

    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.default_planner import DefaultSavePlanner

    d = checkpoint_dir(args.save, iteration)
    multi = dist.is_initialized() and dist.get_world_size() > 1
    rank0 = (not dist.is_initialized()) or dist.get_rank() == 0
    with_optim = not args.no_save_optim
    per_rank_rng = bool(getattr(args, "data_parallel_random_init", False)) and not args.no_save_rng
    rng_states = get_rng_state(per_dp_rank=True) if per_rank_rng else None      # collective
    if rank0:
        os.makedirs(d, exist_ok=True)
        common = dict(args=_plain_namespace(args), checkpoint_version=3.0, iteration=iteration,
                      num_floating_point_operations_so_far=flops)
        if with_optim and optimizer is not None:
            common["optimizer"] = dict(step=optimizer.step_count, param_groups=optimizer.param_groups,
                                       sharded=optimizer.sharded, world=optimizer.world, layout=optimizer.layout())
            if opt_param_scheduler is not None:
                common["opt_param_scheduler"] = opt_param_scheduler.state_dict()
        if not args.no_save_rng:
            common["rng_state"] = rng_states if rng_states is not None else get_rng_state()
        _atomic_save(common, os.path.join(d, DIST_COMMON))
        with open(os.path.join(d, DIST_META + ".tmp"), "w") as f:
            json.dump(dict(sharded_backend=args.dist_ckpt_format, sharded_backend_version=1, common_backend="torch",
                           common_backend_version=1), f)
        os.replace(os.path.join(d, DIST_META + ".tmp"), os.path.join(d, DIST_META))
    _barrier()
    tensors = _dist_tensor_dict(model, optimizer, args, with_optim)
    # replicated tensors are written once: by the lowest rank that holds them, or spread over all holders
    planner = DefaultSavePlanner(dedup_save_to_lowest_rank=not args.ckpt_fully_parallel_save)
    group = mpu.get_transformer_model_group() if multi else None
    dcp.save(tensors, checkpoint_id=d, planner=planner, process_group=group, no_dist=not multi)
    return d


def _load_dist(d, model, optimizer, args, want_optim: bool):
    import torch.distributed.checkpoint as dcp

    multi = dist.is_initialized() and dist.get_world_size() > 1
    common = torch.load(os.path.join(d, DIST_COMMON), map_location="cpu", weights_only=False)
    opt_meta = common.get("optimizer")
    load_optim = bool(want_optim and optimizer is not None and opt_meta is not None)
    if load_optim:
        if opt_meta["layout"] != optimizer.layout() or opt_meta.get("world") != optimizer.world or \
                bool(opt_meta.get("sharded")) != bool(optimizer.sharded):
            raise RuntimeError("the distributed checkpoint's optimizer shares were written under another layout "
                               "(data-parallel size, bucket size or model); resume with the same layout, convert "
                               "through a non-distributed checkpoint, or use --no-load-optim")
    inner = model.module if hasattr(model, "module") else model
    want = _dist_tensor_dict(model, optimizer, args, load_optim)
    target = {k: torch.empty_like(v, device="cpu") for k, v in want.items()}
    dcp.load(target, checkpoint_id=d, process_group=mpu.get_transformer_model_group() if multi else None,
             no_dist=not multi)
    sd = {}
    for k, v in target.items():
        if k.startswith("model."):
            sd[k[len("model."):].split("@tp")[0]] = v
    inner.load_state_dict(sd, strict=True)
    if load_optim:
        for k, v in target.items():
            if k.startswith("optimizer."):
                _, kind, rest = k.split(".", 2)
                i = int(rest.split("@")[0][len("region"):])
                getattr(optimizer, kind)[i].copy_(v)
        optimizer.step_count = opt_meta["step"]
        optimizer.param_groups[0].update(opt_meta["param_groups"][0])
    return common, load_optim


# ----------------------------------------------------------------------------- save
def save_checkpoint(iteration: int, model, optimizer, opt_param_scheduler, args,
                    num_floating_point_operations_so_far: float = 0.0) -> Optional[str]:
    root = args.save
    assert root, "--save is not set"
    if getattr(args, "use_dist_ckpt", False):
        path = _save_dist(iteration, model, optimizer, opt_param_scheduler, args, num_floating_point_operations_so_far)
        _barrier()
        if (not dist.is_initialized()) or dist.get_rank() == 0:
            tmp = tracker_filename(root) + ".tmp"
            with open(tmp, "w") as f:
                f.write(str(iteration))
            os.replace(tmp, tracker_filename(root))
        _barrier()
        return path
    dp_rank = mpu.get_data_parallel_rank(with_context_parallel=True)
    sharded_opt = optimizer is not None and getattr(optimizer, "sharded", False) and not args.no_save_optim
    zero2 = sharded_opt and bool(getattr(args, "use_zero2", False))
    if zero2:
        # --use-zero2: every rank writes its own optimizer shares, nothing is gathered
        # (zero2_optim_dp{d}_cp{c}.pt beside the model file, teletron/train/checkpoint/utils.py:88-95)
        _atomic_save(optimizer.state_dict(), zero2_shard_name(root, iteration))
    full_opt = optimizer.gather_full_state() if (sharded_opt and not zero2) else None  # collective: every rank calls it
    per_rank_rng = bool(getattr(args, "data_parallel_random_init", False)) and not args.no_save_rng
    rng_states = get_rng_state(per_dp_rank=True) if per_rank_rng else None  # collective too
    path = None
    if dp_rank == 0:
        sd = dict(args=_plain_namespace(args), checkpoint_version=3.0, iteration=iteration,
                  num_floating_point_operations_so_far=num_floating_point_operations_so_far)
        inner = model.module if hasattr(model, "module") else model
        sd["model"] = {k: v.detach().cpu() for k, v in inner.state_dict().items()}
        if not args.no_save_optim:
            if optimizer is not None and not sharded_opt:
                sd["optimizer"] = optimizer.state_dict()
            elif optimizer is not None:
                sd["optimizer"] = dict(step=optimizer.step_count, param_groups=optimizer.param_groups,
                                       sharded=True, zero2=zero2)
            if opt_param_scheduler is not None:
                sd["opt_param_scheduler"] = opt_param_scheduler.state_dict()
        if not args.no_save_rng:
            sd["rng_state"] = rng_states if rng_states is not None else get_rng_state()
        path = checkpoint_name(root, iteration)
        _atomic_save(sd, path)
        if sharded_opt and full_opt is not None:
            _atomic_save(full_opt, checkpoint_name(root, iteration, filename=DISTOPT_FILE))
    _barrier()
    if (not dist.is_initialized()) or dist.get_rank() == 0:
        os.makedirs(root, exist_ok=True)
        tmp = tracker_filename(root) + ".tmp"
        with open(tmp, "w") as f:
            f.write(str(iteration))
        os.replace(tmp, tracker_filename(root))
    _barrier()
    return path


# ----------------------------------------------------------------------------- load
def load_checkpoint(model, optimizer, opt_param_scheduler, args, strict: bool = True,
                    defer_rng: bool = False) -> Tuple[int, float]:
    """Returns (iteration, num_floating_point_operations_so_far); (0, 0) when nothing was loaded.
    With ``defer_rng`` the saved RNG state is left in ``args.deferred_rng_state`` for the caller to
    apply (``set_rng_state``) once everything that draws random numbers during start-up — data-loader
    worker seeds, for instance — has been constructed."""
    root = args.load
    finetune = args.finetune
    if (not root or not os.path.exists(tracker_filename(root))) and args.pretrained_checkpoint:
        root, finetune = args.pretrained_checkpoint, True
    if not root:
        return 0, 0.0
    try:
        iteration, release = read_tracker(root)
    except FileNotFoundError:
        if args.exit_on_missing_checkpoint:
            print(f">> no checkpoint tracker in {root}; exiting as requested", flush=True)
            _barrier()
            sys.exit(0)
        print(f"WARNING: no checkpoint tracker in {root}; starting from scratch", flush=True)
        return 0, 0.0
    if args.ckpt_step is not None:
        iteration, release = args.ckpt_step, False
    dist_fmt = is_dist_checkpoint(root, iteration, release)
    if dist_fmt and not (getattr(args, "use_dist_ckpt", False) or getattr(args, "auto_detect_ckpt_format", False)):
        raise RuntimeError(f"{checkpoint_dir(root, iteration, release)} holds a distributed checkpoint; pass "
                           "--use-dist-ckpt or --auto-detect-ckpt-format")
    if dist_fmt:
        want_optim = not (finetune or release or args.no_load_optim)
        sd, optim_loaded = _load_dist(checkpoint_dir(root, iteration, release), model, optimizer, args, want_optim)
        if optim_loaded:
            sd.pop("optimizer", None)              # already placed; what is left is read like the plain format
            sd["_optimizer_placed"] = True
    else:
        path = checkpoint_name(root, iteration, release)
        if not os.path.exists(path):
            raise FileNotFoundError(f"checkpoint file {path} is missing or incomplete")
        try:
            sd = torch.load(path, map_location="cpu", weights_only=False)
        except Exception as e:
            raise RuntimeError(f"could not read checkpoint {path}: {e}") from e
        inner = model.module if hasattr(model, "module") else model
        inner.load_state_dict(sd["model"], strict=strict)
    flops = float(sd.get("num_floating_point_operations_so_far", 0.0))
    if finetune or release:
        iteration = 0
        if optimizer is not None:
            optimizer.reload_model_params()
    else:
        iteration = sd.get("iteration", sd.get("total_iters", 0))
        saved = sd.get("args")
        if saved is not None:
            args.consumed_train_samples = getattr(saved, "consumed_train_samples", 0)
            args.consumed_valid_samples = getattr(saved, "consumed_valid_samples", 0)
        if optimizer is not None:
            if sd.get("_optimizer_placed"):
                pass                               # a distributed checkpoint: every rank has read its own shares
            elif not args.no_load_optim and "optimizer" in sd:
                opt_sd = sd["optimizer"]
                if opt_sd.get("zero2"):          # one file per DP x CP rank, each rank reads its own
                    shard = zero2_shard_name(root, iteration)
                    if not os.path.exists(shard):
                        raise FileNotFoundError(f"{shard} is missing: ZeRO-2 optimizer shards can only be read by a "
                                                "run with the same data- and context-parallel sizes")
                    optimizer.load_state_dict(torch.load(shard, map_location="cpu", weights_only=False))
                elif opt_sd.get("sharded"):      # the fp32 state lives beside the model file, in buffer order
                    full = _load_mapped(checkpoint_name(root, iteration, filename=DISTOPT_FILE))
                    optimizer.scatter_full_state(full)
                elif "master" in opt_sd:
                    # a replicated optimizer's regions, one after the other, are the full buffer as well: any
                    # sharding of this run takes its shares from it
                    full = {k: torch.cat([t.reshape(-1) for t in opt_sd[k]]) for k in ("master", "exp_avg", "exp_avg_sq")}
                    full["layout"] = opt_sd.get("layout")
                    optimizer.scatter_full_state(full)
                else:
                    raise RuntimeError("the checkpoint's optimizer entry has no state this optimizer can read; "
                                       "use --no-load-optim")
                optimizer.step_count = opt_sd["step"]
                optimizer.param_groups[0].update(opt_sd["param_groups"][0])
            else:
                optimizer.reload_model_params()
        if opt_param_scheduler is not None and not args.no_load_optim and "opt_param_scheduler" in sd:
            opt_param_scheduler.load_state_dict(sd["opt_param_scheduler"])
        if not args.no_load_rng and "rng_state" in sd:
            if defer_rng:
                args.deferred_rng_state = sd["rng_state"]
            else:
                set_rng_state(sd["rng_state"], _rng_index(args))
    _barrier()
    return iteration, flops
