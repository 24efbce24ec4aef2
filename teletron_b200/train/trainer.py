"""Trainer: ``Trainer(args).pretrain(forward_step_func)``.

Public contract of the reference trainer (teletron/train/trainer.py:66-889): the user passes
``forward_step(data_iterator, model) -> (output, loss_func)`` with
``loss_func(output) -> (loss, {name: value})``; the trainer owns distributed initialisation,
model / optimizer / scheduler construction, the step loop with gradient accumulation,
evaluation, checkpointing, logging, profiling hooks and the branch of encoder ranks into the
producer loop.  One process per GPU; NCCL on GPU, gloo on CPU.
"""
from __future__ import annotations

import datetime
import gc
import math
import os
import random
import sys
import time
from typing import Callable, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..data import build_data_loader, build_dataset
from ..models import build_model
from ..parallel import state as mpu
from ..parallel.ddp import DistributedOptimizer, ParamBuffer
from ..parallel.tp import tp_shard_dims
from . import checkpoint as ckpt
from .arguments import set_args
from .microbatches import BatchSchedule
from .schedule import scheduler_from_args
from .telelog import TrainLogger


class Float16Module(torch.nn.Module):
    """bf16 model wrapper: floating inputs are cast to bf16, the output back to fp32."""

    def __init__(self, module: torch.nn.Module, dtype=torch.bfloat16):
        super().__init__()
        self.module = module.to(dtype)
        self.dtype = dtype

    def forward(self, *args, **kwargs):
        def cast(v):
            return v.to(self.dtype) if torch.is_tensor(v) and v.is_floating_point() and v.dim() > 1 else v

        out = self.module(*[cast(a) for a in args], **{k: cast(v) for k, v in kwargs.items()})
        return out.float() if (torch.is_tensor(out) and not getattr(self.module, "return_local_shard", False)) else out

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)


def _set_random_seed(seed: int, dp_rank: int = 0, per_dp_rank: bool = False):
    s = seed + (10 * dp_rank if per_dp_rank else 0)
    random.seed(s)
    np.random.seed(s)
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(s)


class Trainer:
    def __init__(self, args, build_data: bool = True):
        self.args = args
        set_args(args)
        self.start_time = time.time()
        self._init_distributed()
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.model = self.optimizer = self.opt_param_scheduler = self.buffer = None
        self.train_data_iterator = self.valid_data_iterator = None
        self.num_floating_point_operations_so_far = 0.0
        if mpu.is_encoder_rank():
            # encoder ranks never train: they serve embeddings until the consumers finish
            from ..data.encoder_service import producer_process

            producer_process(args)
            self._shutdown()
            sys.exit(0)
        _set_random_seed(args.seed, mpu.get_data_parallel_rank(), args.data_parallel_random_init)
        self.setup_model_and_optimizer()
        self.logger = TrainLogger(args, TrainLogger.make_writer(args))
        self.timers = None
        if getattr(args, "timing_log_level", 0) > 0 or getattr(args, "log_timers_to_tensorboard", False):
            from .profiling import DeviceTimers

            self.timers = DeviceTimers()
        if build_data:
            self.build_data_iterators()
        self._signal_seen = False
        if getattr(args, "exit_signal_handler", False):
            import signal

            def _on_sigterm(signum, frame):   # acted on between steps, so no kernel or collective is cut short
                self._signal_seen = True

            self._prev_sigterm = signal.signal(signal.SIGTERM, _on_sigterm)
        if getattr(args, "deferred_rng_state", None) is not None:
            # after everything that consumes start-up randomness
            ckpt.set_rng_state(args.deferred_rng_state, ckpt._rng_index(args))
            args.deferred_rng_state = None

    # ------------------------------------------------------------------ distributed
    def _init_distributed(self):
        a = self.args
        if torch.cuda.is_available():
            torch.cuda.set_device(a.local_rank % torch.cuda.device_count())
        backend = a.distributed_backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if not dist.is_initialized() and (a.world_size > 1 or "MASTER_PORT" in os.environ):
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group(backend=backend, rank=a.rank, world_size=a.world_size,
                                    timeout=datetime.timedelta(minutes=a.distributed_timeout_minutes))
        if dist.is_initialized():
            mpu.initialize_model_parallel(a.tensor_model_parallel_size, a.pipeline_model_parallel_size,
                                          a.context_parallel_size, a.distributed_vae_world_size,
                                          a.consumer_models_num,
                                          timeout=datetime.timedelta(minutes=a.distributed_timeout_minutes),
                                          expert_model_parallel_size=getattr(a, "expert_model_parallel_size", 1))
            if not mpu.is_encoder_rank():
                mpu.warm_up_groups()       # communicators exist before the model takes the memory
            # agree on the earliest start time for --exit-duration-in-mins (trainer.py:87-92)
            t = torch.tensor([self.start_time], dtype=torch.float64,
                             device="cuda" if backend == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            self.start_time = float(t.item())

    def _shutdown(self):
        # an early exit (--exit-interval, --exit-duration-in-mins, SIGTERM) leaves encoder ranks mid-stream: ask them to
        # stop and drain what they already sent, or they would never reach the barrier below
        it = getattr(self, "train_data_iterator", None)
        if hasattr(it, "close") and self.args.iteration < (self.args.train_iters or 0):
            it.close()
        if dist.is_initialized():
            try:
                dist.barrier()
            except Exception:
                pass

    # ------------------------------------------------------------------ model / optimizer
    def setup_model_and_optimizer(self):
        a = self.args
        if getattr(a, "init_on_device", False) and self.device.type == "cuda":
            with torch.device(self.device):
                model = build_model(a.model, a)
        else:
            model = build_model(a.model, a).to(self.device)
        if a.bf16:
            model = Float16Module(model)
        self.model = model
        inner = model.module if isinstance(model, Float16Module) else model
        group = mpu.get_data_parallel_group(with_context_parallel=True)
        world = mpu.get_data_parallel_world_size(with_context_parallel=True)
        arena = None
        want_fused = a.fused_comm != "off" and a.use_distributed_optimizer and world > 1 and self.device.type == "cuda"
        if want_fused:
            from ..dist import SymmetricArena, symmetric_memory_available

            single_box = a.world_size <= torch.cuda.device_count()
            if symmetric_memory_available() and (single_box or a.fused_comm == "on"):
                try:
                    arena = SymmetricArena(group)
                except Exception as e:
                    if a.fused_comm == "on":
                        raise
                    print(f"WARNING: symmetric memory unavailable ({e}); using NCCL collectives", flush=True)
        self.arena = arena
        cp_ctx = getattr(inner, "cp", None)
        if (a.fused_comm != "off" and cp_ctx is not None and cp_ctx.size > 1 and self.device.type == "cuda"
                and a.world_size <= torch.cuda.device_count()):
            from ..dist import SymmetricArena, symmetric_memory_available
            from ..parallel.fused_ulysses import FusedUlysses

            if symmetric_memory_available():
                try:
                    cp_ctx.fused = FusedUlysses(SymmetricArena(mpu.get_context_parallel_group()))
                    cp_ctx.fused.poison = bool(getattr(a, "poison_comm_buffers", False))
                except Exception as e:
                    if a.fused_comm == "on":
                        raise
                    print(f"WARNING: fused Ulysses unavailable ({e}); using NCCL all-to-all", flush=True)
        tp_ctx = getattr(inner, "tp", None)
        if (a.fused_comm != "off" and tp_ctx is not None and tp_ctx.size > 1 and self.device.type == "cuda"
                and a.world_size <= torch.cuda.device_count()):
            from ..dist import SymmetricArena, symmetric_memory_available
            from ..parallel.tp import FusedTP

            if symmetric_memory_available():
                try:
                    tp_ctx.fused = FusedTP(SymmetricArena(mpu.get_tensor_model_parallel_group()))
                except Exception as e:
                    if a.fused_comm == "on":
                        raise
                    print(f"WARNING: fused tensor-parallel kernels unavailable ({e}); using NCCL collectives", flush=True)
        tp_names = tuple(tp_shard_dims(inner, params=True)) if a.tensor_model_parallel_size > 1 else None
        if arena is not None:
            torch.cuda.empty_cache()     # the fp32 blocks of the initialisation: the arena is allocated outside this cache
        self.buffer = ParamBuffer(inner, shard_world=world if a.use_distributed_optimizer else 1, arena=arena,
                                  bucket_size=getattr(a, "ddp_bucket_size", None), tp_sharded_names=tp_names)
        # the peer-memory path overlaps each bucket's reduction with backward by default; NCCL on request
        overlap = world > 1 and (a.overlap_grad_reduce or (arena is not None and a.overlap_grad_reduce is not False))
        self.optimizer = DistributedOptimizer(
            self.buffer, group if world > 1 else None, lr=a.lr, betas=(a.adam_beta1, a.adam_beta2),
            eps=a.adam_eps, weight_decay=a.weight_decay, clip_grad=a.clip_grad,
            sharded=a.use_distributed_optimizer, grad_scale=1.0 / max(a.data_parallel_size, 1),
            tp_group=mpu.get_tensor_model_parallel_group() if a.tensor_model_parallel_size > 1 else None,
            tp_sharded_names=tp_names or (), overlap=overlap, kind=getattr(a, "optimizer", "adam"),
            momentum=getattr(a, "sgd_momentum", 0.9))
        self.optimizer.log_num_zeros = bool(getattr(a, "log_num_zeros_in_grad", False))
        self.opt_param_scheduler = scheduler_from_args(a, self.optimizer) if (a.train_iters or a.train_samples) else None
        if a.load or a.pretrained_checkpoint:
            a.iteration, self.num_floating_point_operations_so_far = ckpt.load_checkpoint(
                self.model, self.optimizer, self.opt_param_scheduler, a, defer_rng=True)
        if world > 1 and not (a.load or a.pretrained_checkpoint):
            # identical initial weights on every replica (DDP.broadcast_params in the reference)
            dist.broadcast(self.buffer.params, src=mpu.get_group_ranks("dp_cp")[0], group=group)
            self.optimizer.reload_model_params()
        if self.device.type == "cuda":
            # the parameters moved into the flat buffer: their first storages (30 GiB for a 16 B-parameter model) sit in
            # the allocator's cache as odd-sized blocks; hand them back before the first step sizes its own
            torch.cuda.empty_cache()

    # ------------------------------------------------------------------ data
    def build_data_iterators(self):
        a = self.args
        if a.distributed_vae:
            from ..data.batch_loader import create_batch_loader

            self.train_data_iterator = create_batch_loader(a.model, a)
            self.valid_data_iterator = None
            return
        h, w = a.video_resolution
        i2v = (a.task_type == "i2v")
        synthetic = a.synthetic_latents or a.dataset_type == "SyntheticLatentDataset"
        name = "SyntheticLatentDataset" if synthetic else a.dataset_type
        kw = dict(num_frames=a.num_frames, height=h, width=w, i2v=i2v, seed=a.seed, data_path=getattr(a, "data_path", None),
                  min_length=(a.train_iters or 0) * a.global_batch_size)    # finite datasets repeat up to this
        if name == "SyntheticLatentDataset" and "Hunyuan" in a.model:
            name = "SyntheticHunyuanDataset"                  # same role, the HunyuanVideo batch schema
            cfg = (self.model.module if hasattr(self.model, "module") else self.model).cfg
            kw.update(text_dim=cfg.text_embed_dim, pooled_dim=cfg.pooled_projection_dim, i2v=cfg.in_channels > 16)
        if getattr(a, "text_dim", None):
            kw["text_dim"] = a.text_dim
        if getattr(a, "text_len", None):
            kw["text_len"] = a.text_len
        ds = build_dataset(name, **kw)
        dp_rank, dp_size = mpu.get_data_parallel_rank(), a.data_parallel_size
        dl = build_data_loader(ds, a.consumed_train_samples, a.micro_batch_size, dp_rank, dp_size,
                               a.dataloader_type, a.num_workers, a.seed)
        self.train_data_iterator = iter(dl)
        if a.eval_iters > 0:
            vdl = build_data_loader(ds, a.consumed_valid_samples, a.micro_batch_size, dp_rank, dp_size,
                                    "single", 0, a.seed + 1)
            self.valid_data_iterator = iter(vdl)

    def _set_batch_level(self, strict: bool):
        """Global batch and micro-batch count for the samples consumed so far (constant unless
        ``--rampup-batch-size`` is given), mirrored into the arguments the rest of the loop reads."""
        a = self.args
        if getattr(self, "batch_schedule", None) is None:
            self.batch_schedule = BatchSchedule(a.global_batch_size, a.micro_batch_size, a.data_parallel_size,
                                                getattr(a, "rampup_batch_size", None))
        self.batch_schedule.update(a.consumed_train_samples, strict=strict)
        a.num_micro_batches = self.batch_schedule.num_micro_batches
        a.current_global_batch_size = self.batch_schedule.current_global_batch_size

    # ------------------------------------------------------------------ one step
    def train_step(self, forward_step_func: Callable, data_iterator=None):
        """Forward/backward over the micro-batches, gradient reduction, optimizer and schedule step.
        Returns (loss_dict, skipped_iter, grad_norm, num_zeros_in_grad)."""
        a = self.args
        it = data_iterator if data_iterator is not None else self.train_data_iterator
        self.model.train()
        self.optimizer.zero_grad()
        n_mb = a.num_micro_batches
        reduced_all = []
        tm = getattr(self, "timers", None)
        fine = tm is not None and a.timing_log_level >= 2
        if tm is not None:
            tm.start("forward-backward")
        for mb in range(n_mb):
            if mb == n_mb - 1:
                self.optimizer.begin_last_microbatch()     # bucket reductions may start during this backward
            if fine:
                tm.start("forward-compute")
            output, loss_func = forward_step_func(it, self.model)
            loss, reduced = loss_func(output)
            if fine:
                tm.stop("forward-compute")
                tm.start("backward-compute")
            (loss / n_mb).backward()
            if fine:
                tm.stop("backward-compute")
            reduced_all.append(reduced)
        if tm is not None:
            tm.stop("forward-backward")
            tm.start("grads-reduce")
        if a.empty_unused_memory_level >= 2 and self.device.type == "cuda":
            torch.cuda.empty_cache()
        self.optimizer.reduce_gradients()
        if tm is not None:
            tm.stop("grads-reduce")
            tm.start("optimizer")
        ok, grad_norm, num_zeros = self.optimizer.step()
        if tm is not None:
            tm.stop("optimizer")
        if a.empty_unused_memory_level >= 1 and self.device.type == "cuda":
            torch.cuda.empty_cache()
        if ok and self.opt_param_scheduler is not None:
            self.opt_param_scheduler.step(increment=getattr(a, "current_global_batch_size", a.global_batch_size))
        loss_dict = {}
        for k in (reduced_all[0] or {}):
            vals = [r[k] for r in reduced_all]
            loss_dict[k] = sum(v if torch.is_tensor(v) else torch.tensor(v) for v in vals) / len(vals)
        if a.check_for_nan_in_loss_and_grad:
            bad = [k for k, v in loss_dict.items() if not math.isfinite(float(v))]
            if grad_norm is not None and not math.isfinite(float(grad_norm)):
                bad.append("grad_norm")
            if bad:
                raise RuntimeError(f"non-finite {', '.join(bad)} at iteration {a.iteration + 1} on rank {a.rank} "
                                   "(--check-for-nan-in-loss-and-grad)")
        return loss_dict, (0 if ok else 1), grad_norm, num_zeros

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate(self, forward_step_func: Callable, data_iterator=None, iters: Optional[int] = None):
        a = self.args
        it = data_iterator if data_iterator is not None else self.valid_data_iterator
        if it is None:
            return {}
        self.model.eval()
        total = {}
        n = iters if iters is not None else a.eval_iters
        for _ in range(n):
            output, loss_func = forward_step_func(it, self.model)
            _, reduced = loss_func(output)
            for k, v in reduced.items():
                total[k] = total.get(k, 0.0) + float(v)
            a.consumed_valid_samples += a.global_batch_size
        self.model.train()
        return {k: v / max(n, 1) for k, v in total.items()}

    # ------------------------------------------------------------------ main loop
    def pretrain(self, forward_step_func: Callable):
        a = self.args
        if not a.skip_train and a.train_iters and a.iteration < a.train_iters:
            self.train(forward_step_func)
        if a.eval_iters > 0 and self.valid_data_iterator is not None:
            res = self.evaluate(forward_step_func)
            self.logger.log_validation(res, a.iteration, prefix=f"the end of training (iteration {a.iteration})")
        if a.save and a.iteration != 0 and not getattr(self, "_saved_at", None) == a.iteration:
            self.save(a.iteration)
        self._shutdown()

    def save(self, iteration):
        ckpt.save_checkpoint(iteration, self.model, self.optimizer, self.opt_param_scheduler, self.args,
                             self.num_floating_point_operations_so_far)
        self._saved_at = iteration

    def train(self, forward_step_func: Callable):
        a = self.args
        iteration = a.iteration
        tokens_per_step = getattr(a, "tokens_per_sample", 0) * a.global_batch_size
        prof = None
        if a.consumer_profile:
            from .profiling import make_torch_profiler

            prof = make_torch_profiler(a, "consumer")
            prof.__enter__()
        if a.manual_gc:
            gc.disable()
            gc.collect()
        use_events = torch.cuda.is_available()
        from .profiling import MemorySnapshot, ProfileWindow

        window = ProfileWindow(a)
        mem_snap = MemorySnapshot(a.rank)
        n_mb_prev = a.num_micro_batches
        first_step = True
        while iteration < a.train_iters:
            # batch-size ramp-up: a new level starts from a checkpoint, then has to split into micro-batches
            self._set_batch_level(strict=False)
            if a.num_micro_batches != n_mb_prev and iteration != 0:
                if a.num_micro_batches < n_mb_prev:
                    raise RuntimeError("the number of micro-batches shrank during batch-size ramp-up")
                if a.save:
                    self.save(iteration)
            n_mb_prev = a.num_micro_batches
            self._set_batch_level(strict=True)
            tokens_per_step = getattr(a, "tokens_per_sample", 0) * a.current_global_batch_size
            window.before_step(iteration)
            mem_snap.begin()
            if use_events:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            loss_dict, skipped, grad_norm, num_zeros = self.train_step(forward_step_func)
            dev_ms = 0.0
            if use_events:
                e1.record()
                e1.synchronize()
                dev_ms = e0.elapsed_time(e1)
                from ..ops import _lib

                if _lib.available():
                    _lib.check_status()
            mem_snap.dump(iteration)
            if first_step and self.device.type == "cuda":
                # the first step's one-off allocations leave cached blocks that nothing reuses: hand them back once,
                # so that allocations outside the caching allocator (NCCL buffers made at a group's or a peer's first
                # use, growth of the symmetric arena) still find memory next to a model that fills the GPU
                torch.cuda.empty_cache()
            first_step = False
            iteration += 1
            a.iteration = iteration
            a.consumed_train_samples += a.current_global_batch_size
            lr = self.optimizer.param_groups[0]["lr"]
            params_norm = self.buffer.params.float().norm() if a.log_params_norm else None
            self.logger.log(loss_dict, iteration, lr, 1.0, grad_norm, skipped, params_norm,
                            tokens=tokens_per_step, device_ms=dev_ms, timers=self.timers, num_zeros_in_grad=num_zeros)
            if prof is not None:
                prof.step()
            window.after_step(iteration)
            if a.manual_gc and a.manual_gc_interval and iteration % a.manual_gc_interval == 0:
                gc.collect()
            if a.eval_interval and a.eval_iters > 0 and iteration % a.eval_interval == 0:
                if a.manual_gc and a.manual_gc_eval:
                    gc.collect()          # evaluation allocates differently: start and leave it with a clean heap
                res = self.evaluate(forward_step_func)
                if a.manual_gc and a.manual_gc_eval:
                    gc.collect(generation=0)
                if a.empty_unused_memory_level >= 1 and self.device.type == "cuda":
                    torch.cuda.empty_cache()
                self.logger.log_validation(res, iteration)
            if a.save and a.save_interval and iteration % a.save_interval == 0:
                self.save(iteration)
            if a.exit_signal_handler:
                flag = torch.tensor([int(self._signal_seen)], device=self.device)
                if dist.is_initialized():
                    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=mpu.get_transformer_model_group())
                if int(flag.item()):        # any rank got SIGTERM: everybody saves and leaves together
                    if a.save:
                        self.save(iteration)
                    print(f"exiting at iteration {iteration}: termination signal received", flush=True)
                    break
            if a.exit_duration_in_mins:
                mins = (time.time() - self.start_time) / 60.0
                flag = torch.tensor([int(mins > a.exit_duration_in_mins)], device=self.device)
                if dist.is_initialized():
                    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=mpu.get_transformer_model_group())
                if int(flag.item()):
                    if a.save:
                        self.save(iteration)
                    print(f"exiting after {mins:.1f} minutes at iteration {iteration}", flush=True)
                    break
            if a.exit_interval and iteration % a.exit_interval == 0:
                if a.save:
                    self.save(iteration)
                print(f"exiting at iteration {iteration} (--exit-interval)", flush=True)
                break
        if prof is not None:
            prof.__exit__(None, None, None)
        return iteration
