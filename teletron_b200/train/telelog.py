"""Training-loop logging: loss accumulation between log intervals, skipped / NaN iteration
counters, TensorBoard scalars on the last rank and one console line per interval
(teletron/train/telelogger.py:18-262).  In addition it reports device-timed throughput in
tokens/s, which the reference never logs.
"""
from __future__ import annotations

import math
import time
from typing import Dict, Optional

import torch
import torch.distributed as dist


def _log_rank(args) -> int:
    """The rank that prints: the last one that runs the transformer (encoder ranks sit behind it and never log)."""
    enc = int(getattr(args, "distributed_vae_world_size", 0) or 0) if getattr(args, "distributed_vae", False) else 0
    return args.world_size - 1 - enc


class _TeeWriter:
    """``add_scalar`` to TensorBoard (when present) and to a Weights & Biases run."""

    def __init__(self, tb, wb_run):
        self.tb, self.wb = tb, wb_run

    def add_scalar(self, tag, value, step):
        if self.tb is not None:
            self.tb.add_scalar(tag, value, step)
        self.wb.log({tag: value}, step=int(step))

    def flush(self):
        if self.tb is not None:
            self.tb.flush()

    def close(self):
        if self.tb is not None:
            self.tb.close()
        self.wb.finish()


class TrainLogger:
    ADV, SKIP, NAN = "advanced iterations", "skipped iterations", "nan iterations"

    def __init__(self, args, writer=None):
        self.args = args
        self.writer = writer
        self.totals: Dict[str, float] = {}
        self.counts = {self.ADV: 0, self.SKIP: 0, self.NAN: 0}
        self.t_last = time.time()
        self.tokens_since = 0
        self.device_ms_since = 0.0
        self.reported_memory = False

    @staticmethod
    def make_writer(args):
        """Scalar writer on the last rank only (teletron/utils/config.py:59-70): a TensorBoard ``SummaryWriter``
        when ``--tensorboard-dir`` is given, mirrored to Weights & Biases when ``--wandb-project`` is given and the
        package is installed (the reference declares that mirror but never creates it, utils/config.py:42-45)."""
        if args.rank != _log_rank(args):
            return None
        tb = wb = None
        if args.tensorboard_dir:
            try:
                from torch.utils.tensorboard import SummaryWriter

                tb = SummaryWriter(log_dir=args.tensorboard_dir, max_queue=args.tensorboard_queue_size)
            except Exception as e:  # tensorboard missing: keep training
                print(f"WARNING: TensorBoard unavailable ({e})", flush=True)
        if getattr(args, "wandb_project", ""):
            try:
                import wandb

                wb = wandb.init(project=args.wandb_project, name=getattr(args, "wandb_exp_name", "") or None,
                                dir=getattr(args, "wandb_save_dir", "") or None,
                                config={k: v for k, v in vars(args).items()
                                        if isinstance(v, (int, float, str, bool, type(None)))})
            except Exception as e:
                print(f"WARNING: Weights & Biases unavailable ({e})", flush=True)
        if wb is None:
            return tb
        return _TeeWriter(tb, wb)

    def log(self, loss_dict, iteration, lr, loss_scale, grad_norm, skipped_iter, params_norm=None,
            tokens: int = 0, device_ms: float = 0.0, timers=None, num_zeros_in_grad=None) -> bool:
        """``timers``: a ``DeviceTimers`` whose intervals since the last report are summarised (collectively: every
        rank must pass it) at the log interval, printed as ``name: ms per iteration`` and, with
        ``--log-timers-to-tensorboard``, written as ``<name>-time`` scalars."""
        a = self.args
        self.counts[self.SKIP if skipped_iter else self.ADV] += 1
        got_nan = False
        for k, v in loss_dict.items():
            val = float(v)
            if not skipped_iter:
                self.totals[k] = self.totals.get(k, 0.0) + val
            got_nan |= math.isnan(val) or math.isinf(val)
        self.counts[self.NAN] += int(got_nan)
        self.tokens_since += tokens
        self.device_ms_since += device_ms
        w = self.writer
        if w is not None and iteration % a.tensorboard_log_interval == 0:
            samples = a.consumed_train_samples
            w.add_scalar("learning-rate", lr, iteration)
            w.add_scalar("learning-rate vs samples", lr, samples)
            w.add_scalar("batch-size", getattr(a, "current_global_batch_size", a.global_batch_size), iteration)
            for k, v in loss_dict.items():
                w.add_scalar(k, float(v), iteration)
                w.add_scalar(k + " vs samples", float(v), samples)
            w.add_scalar("loss-scale", float(loss_scale), iteration)
            w.add_scalar("world-size", a.world_size, iteration)
            if grad_norm is not None:
                w.add_scalar("grad-norm", float(grad_norm), iteration)
            if num_zeros_in_grad is not None:
                w.add_scalar("num-zeros", float(num_zeros_in_grad), iteration)
                w.add_scalar("num-zeros vs samples", float(num_zeros_in_grad), samples)
            if params_norm is not None:
                w.add_scalar("params-norm", float(params_norm), iteration)
            if a.log_memory_to_tensorboard and torch.cuda.is_available():
                ms = torch.cuda.memory_stats()
                w.add_scalar("mem-reserved-bytes", ms["reserved_bytes.all.current"], iteration)
                w.add_scalar("mem-allocated-bytes", ms["allocated_bytes.all.current"], iteration)
        if iteration % a.log_interval != 0:
            return False
        n_adv = max(self.counts[self.ADV], 1)
        elapsed = time.time() - self.t_last
        n_iters = max(self.counts[self.ADV] + self.counts[self.SKIP], 1)
        batch = getattr(a, "current_global_batch_size", a.global_batch_size)
        parts = [f"iteration {iteration:8d}/{a.train_iters or 0:8d}",
                 f"consumed samples: {a.consumed_train_samples:12d}",
                 f"elapsed time per iteration (ms): {elapsed * 1000.0 / n_iters:.1f}",
                 f"learning rate: {lr:.3E}", f"global batch size: {batch:5d}"]
        for k, tot in self.totals.items():
            parts.append(f"{k}: {tot / n_adv:.6E}")
        parts.append(f"loss scale: {float(loss_scale):.1f}")
        if grad_norm is not None:
            parts.append(f"grad norm: {float(grad_norm):.3f}")
        if num_zeros_in_grad is not None:
            parts.append(f"num zeros: {float(num_zeros_in_grad):.1f}")
        if params_norm is not None:
            parts.append(f"params norm: {float(params_norm):.3f}")
        if self.device_ms_since > 0:
            tps = self.tokens_since / (self.device_ms_since * 1e-3)
            parts.append(f"tokens/s (device-timed): {tps:.1f}")
            if w is not None:
                w.add_scalar("tokens-per-second", tps, iteration)
        parts.append(f"number of skipped iterations: {self.counts[self.SKIP]:3d}")
        parts.append(f"number of nan iterations: {self.counts[self.NAN]:3d}")
        if a.rank == _log_rank(a):
            print(" | ".join(parts), flush=True)
        if timers is not None:
            n_it = max(self.counts[self.ADV] + self.counts[self.SKIP], 1)
            from ..parallel import state as mpu

            grp = mpu.get_transformer_model_group() if mpu.model_parallel_is_initialized() else None
            per_it = {k: v / n_it for k, v in timers.summary(group=grp).items()}   # encoder ranks take no part
            self.last_timings = per_it
            if a.rank == _log_rank(a) and per_it:
                print("    time (ms) | " + " | ".join(f"{k}: {v:.2f}" for k, v in per_it.items()), flush=True)
            if w is not None and a.log_timers_to_tensorboard:
                for k, v in per_it.items():
                    w.add_scalar(f"{k}-time", v, iteration)
        report_mem = not self.reported_memory and torch.cuda.is_available()
        if report_mem:
            self.reported_memory = True
            if a.rank == _log_rank(a):
                mb = 1024.0 * 1024.0
                print(f"[rank {a.rank}] memory (MB) | allocated: {torch.cuda.memory_allocated() / mb:.0f}"
                      f" | max allocated: {torch.cuda.max_memory_allocated() / mb:.0f}"
                      f" | reserved: {torch.cuda.memory_reserved() / mb:.0f}", flush=True)
        self.totals = {}
        self.counts = {k: 0 for k in self.counts}
        self.tokens_since, self.device_ms_since = 0, 0.0
        self.t_last = time.time()
        return report_mem

    def log_validation(self, loss_dict, iteration, prefix: str = None):
        """Framed console line on the last rank (each value with its perplexity ``exp(min(20, value))``, as the
        reference prints, teletron/train/trainer.py:776-795) and the validation scalars (telelogger.py:256-262)."""
        a = self.args
        if a.rank == _log_rank(a) and loss_dict:
            line = f" validation loss at {prefix or f'iteration {iteration}'} | "
            for k, v in loss_dict.items():
                line += f"{k} value: {float(v):.6E} | {k} PPL: {math.exp(min(20.0, float(v))):.6E} | "
            bar = "-" * (len(line) + 1)
            print(f"{bar}\n{line}\n{bar}", flush=True)
        if self.writer is None:
            return
        for k, v in loss_dict.items():
            self.writer.add_scalar(f"{k} validation", float(v), iteration)
            self.writer.add_scalar(f"{k} validation vs samples", float(v), a.consumed_train_samples)
            self.writer.add_scalar(f"{k} validation ppl", math.exp(min(20.0, float(v))), iteration)
