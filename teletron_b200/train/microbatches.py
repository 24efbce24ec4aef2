"""Number of micro-batches per optimizer step, constant or ramped up with the samples consumed.

``--rampup-batch-size START INCREMENT SAMPLES`` grows the global batch from ``START`` to
``--global-batch-size`` in steps of ``INCREMENT``, spending ``SAMPLES / number_of_increments`` samples on each
level, as the reference's calculators do (teletron/utils/microbatches.py:8-144; the trainer re-evaluates
them every iteration and saves a checkpoint when the level changes, teletron/train/trainer.py:537-545).
Here one ``BatchSchedule`` object covers both cases and the current level is a pure function of the
consumed-sample count, so a resumed run lands on the same level without extra state.
"""
from __future__ import annotations

from typing import Optional, Sequence


class BatchSchedule:
    def __init__(self, global_batch_size: int, micro_batch_size: int, data_parallel_size: int,
                 rampup: Optional[Sequence] = None):
        self.per_pass = int(micro_batch_size) * int(data_parallel_size)  # samples of one micro-batch pass over DP
        if self.per_pass <= 0:
            raise ValueError("micro batch size and data-parallel size must be positive")
        self.final = int(global_batch_size)
        if self.final <= 0:
            raise ValueError("global batch size must be positive")
        self.start, self.increment, self.ramp_samples, self.levels = self.final, 0, 0, 0
        if rampup:
            if len(rampup) != 3:
                raise ValueError("--rampup-batch-size takes <start batch size> <increment> <ramp-up samples>")
            self.start, self.increment, self.ramp_samples = (int(v) for v in rampup)
            span = self.final - self.start
            if self.start <= 0 or self.increment <= 0 or self.ramp_samples < 0 or span < 0:
                raise ValueError(f"bad batch-size ramp {list(rampup)} towards global batch {self.final}")
            if span % self.increment:
                raise ValueError(f"global batch {self.final} - start {self.start} is not a multiple of the "
                                 f"increment {self.increment}")
            self.levels = span // self.increment
        self.current_global_batch_size = None
        self.num_micro_batches = None
        self.update(0, strict=not rampup)

    def global_batch_at(self, consumed_samples: int) -> int:
        if self.levels == 0 or consumed_samples > self.ramp_samples:
            return self.final
        per_level = self.ramp_samples / self.levels
        level = int(consumed_samples / per_level) if per_level > 0 else self.levels
        return min(self.start + level * self.increment, self.final)

    def update(self, consumed_samples: int, strict: bool = True) -> int:
        """Set the level for ``consumed_samples``; with ``strict`` the level must split evenly into
        micro-batch passes (the reference checks this only on its second call per iteration)."""
        g = self.global_batch_at(int(consumed_samples))
        if strict and g % self.per_pass:
            raise ValueError(f"current global batch {g} is not divisible by micro batch x data-parallel size "
                             f"= {self.per_pass}")
        self.current_global_batch_size = g
        self.num_micro_batches = g // self.per_pass
        return self.num_micro_batches


_SCHEDULE: Optional[BatchSchedule] = None


def build_num_microbatches_calculator(args) -> BatchSchedule:
    """Create the process-wide schedule from parsed arguments and mirror its state into them."""
    global _SCHEDULE
    _SCHEDULE = BatchSchedule(args.global_batch_size, args.micro_batch_size, args.data_parallel_size,
                              getattr(args, "rampup_batch_size", None))
    _mirror(args)
    if getattr(args, "rank", 0) == 0 and _SCHEDULE.levels:
        print(f"batch-size ramp-up: {_SCHEDULE.start} -> {_SCHEDULE.final} in steps of {_SCHEDULE.increment} over "
              f"{_SCHEDULE.ramp_samples} samples", flush=True)
    return _SCHEDULE


def _mirror(args):
    args.num_micro_batches = _SCHEDULE.num_micro_batches
    args.current_global_batch_size = _SCHEDULE.current_global_batch_size


def get_num_microbatches() -> int:
    return _SCHEDULE.num_micro_batches


def get_current_global_batch_size() -> int:
    return _SCHEDULE.current_global_batch_size


def update_num_microbatches(consumed_samples: int, consistency_check: bool = True, args=None) -> int:
    n = _SCHEDULE.update(consumed_samples, strict=consistency_check)
    if args is not None:
        _mirror(args)
    return n
