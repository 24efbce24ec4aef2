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
    """Allocator history per training step when the environment names ``MEMORY_SNAPSHOT``: ``begin()`` before the step
    starts the recording, ``dump(iteration)`` after it writes ``memory_<time>_iter<i>_rank<r>.pt`` under
    ``PROF_SAVE_PATH`` and stops the recording (teletron/train/trainer.py:549-567).  ``backend`` is the module
    that provides ``_record_memory_history`` / ``_dump_snapshot`` (``torch.cuda.memory``; a stand-in in tests)."""

    def __init__(self, rank: int, backend=None, max_entries: int = 80000):
        self.backend = backend if backend is not None else (torch.cuda.memory if torch.cuda.is_available() else None)
        self.enabled = bool(os.environ.get("MEMORY_SNAPSHOT")) and self.backend is not None
        self.dir = os.environ.get("PROF_SAVE_PATH", ".")
        self.rank = rank
        self.max_entries = max_entries

    def begin(self):
        if self.enabled:
            self.backend._record_memory_history(max_entries=self.max_entries)

    def dump(self, iteration: int):
        if not self.enabled:
            return None
        os.makedirs(self.dir, exist_ok=True)
        stamp = time.strftime("%Y%m%d_%H%M%S", time.localtime())
        path = os.path.join(self.dir, f"memory_{stamp}_iter{iteration}_rank{self.rank}.pt")
        self.backend._dump_snapshot(path)
        self.backend._record_memory_history(enabled=None)
        return path


from ..utils.nvtx import nvtx_range, set_nvtx  # noqa: E402,F401  (named ranges around the fused kernels)


class ProfileWindow:
    """``--profile``: on the ranks of ``--profile-ranks``, from ``--profile-step-start`` to ``--profile-step-end``
    the CUDA profiler API is started (for an external profiler attached with capture range = cudaProfilerApi),
    autograd emits NVTX ranges for every op and the framework's own ranges around its fused kernels are switched on
    (teletron/train/trainer.py:527-531, 659-662)."""

    def __init__(self, args, cudart=None):
        self.on = bool(args.profile) and args.rank in args.profile_ranks and (cudart is not None or torch.cuda.is_available())
        self.start, self.end = args.profile_step_start, args.profile_step_end
        self._cudart = cudart
        self._emit = None

    def before_step(self, iteration: int):
        if self.on and iteration == self.start and self._emit is None:
            (self._cudart or torch.cuda.cudart()).cudaProfilerStart()
            self._emit = torch.autograd.profiler.emit_nvtx(record_shapes=True)
            self._emit.__enter__()
            set_nvtx(True)

    def after_step(self, iteration: int):
        """``iteration``: number of completed steps."""
        if self.on and iteration == self.end and self._emit is not None:
            set_nvtx(False)
            self._emit.__exit__(None, None, None)
            self._emit = None
            (self._cudart or torch.cuda.cudart()).cudaProfilerStop()


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
