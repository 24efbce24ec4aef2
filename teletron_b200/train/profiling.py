"""Profiling hooks: torch.profiler chrome traces per rank (``--consumer-profile`` /
``--producer-profile``, teletron/train/trainer.py:509-526, distributed_encoder.py:116-136), CUDA
memory-history snapshots when ``MEMORY_SNAPSHOT`` is set (trainer.py:549-567), and CUDA-event
phase timers that report device time as the maximum over ranks.
"""
from __future__ import annotations

import os
import time
from collections import defaultdict

import torch
import torch.distributed as dist


def make_torch_profiler(args, role: str):
    out_dir = os.path.join(args.profile_path, role)
    os.makedirs(out_dir, exist_ok=True)
    start, end = args.profile_step_start, args.profile_step_end
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)

    def on_ready(prof):
        prof.export_chrome_trace(os.path.join(out_dir, f"rank_{args.rank}.json"))

    return torch.profiler.profile(
        activities=acts, record_shapes=True, with_stack=True,
        schedule=torch.profiler.schedule(wait=max(start - 1, 0), warmup=1, active=max(end - start, 1), repeat=1),
        on_trace_ready=on_ready)


class MemorySnapshot:
    """Records allocator history while active and dumps ``memory_<time>_iter<i>_rank<r>.pt``."""

    def __init__(self, rank: int):
        self.enabled = bool(os.environ.get("MEMORY_SNAPSHOT")) and torch.cuda.is_available()
        self.dir = os.environ.get("PROF_SAVE_PATH", ".")
        self.rank = rank
        if self.enabled:
            torch.cuda.memory._record_memory_history(max_entries=100000)

    def dump(self, iteration: int):
        if not self.enabled:
            return None
        os.makedirs(self.dir, exist_ok=True)
        path = os.path.join(self.dir, f"memory_{int(time.time())}_iter{iteration}_rank{self.rank}.pt")
        torch.cuda.memory._dump_snapshot(path)
        return path


class DeviceTimers:
    """Named phase timers: CUDA events on the current stream when a GPU is present (no host synchronisation
    until ``summary``), the wall clock otherwise.  ``summary()`` gives per-name milliseconds summed over the
    recorded intervals, as the maximum over the ranks of ``group``."""

    def __init__(self, use_cuda=None):
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self._open = {}
        self._pairs = defaultdict(list)

    def _mark(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    def start(self, name: str):
        self._open[name] = self._mark()

    def stop(self, name: str):
        self._pairs[name].append((self._open.pop(name), self._mark()))

    def summary(self, group=None, reset: bool = True):
        if self.cuda:
            torch.cuda.synchronize()
        names = sorted(self._pairs)
        span = (lambda a, b: a.elapsed_time(b)) if self.cuda else (lambda a, b: (b - a) * 1e3)
        vals = torch.tensor([sum(span(a, b) for a, b in self._pairs[n]) for n in names], dtype=torch.float64,
                            device="cuda" if (self.cuda and (not dist.is_initialized() or dist.get_backend(group) == "nccl"))
                            else "cpu")
        if dist.is_initialized() and dist.get_world_size(group) > 1 and len(names):
            dist.all_reduce(vals, op=dist.ReduceOp.MAX, group=group)
        if reset:
            self._pairs.clear()
        return dict(zip(names, vals.tolist()))
