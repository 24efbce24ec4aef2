"""Learning-rate and weight-decay schedule, advanced in consumed samples.

Behaviour of the reference scheduler (teletron/train/lr_scheduler.py:30-251): linear warm-up
from ``init_lr`` to ``max_lr`` over ``lr_warmup_steps``; then constant / linear / cosine /
inverse-square-root decay down to ``min_lr`` over ``lr_decay_steps``; weight decay constant or
ramped linearly / by cosine from start to end over ``wd_incr_steps``.  ``step(increment)``
is called with the number of samples of the global batch (teletron/train/trainer.py:742-746).
State-dict keys match so schedules resume from reference checkpoints (old key names accepted).
"""
from __future__ import annotations

import math


class OptimizerParamScheduler:
    def __init__(self, optimizer, init_lr, max_lr, min_lr, lr_warmup_steps, lr_decay_steps, lr_decay_style,
                 start_wd, end_wd, wd_incr_steps, wd_incr_style, use_checkpoint_opt_param_scheduler=True,
                 override_opt_param_scheduler=False):
        self.optimizer = optimizer
        self.init_lr, self.max_lr, self.min_lr = float(init_lr), float(max_lr), float(min_lr)
        assert 0.0 <= self.min_lr <= self.max_lr and self.init_lr <= self.max_lr
        self.lr_warmup_steps, self.lr_decay_steps = lr_warmup_steps, lr_decay_steps
        assert self.lr_decay_steps > 0 and self.lr_warmup_steps < self.lr_decay_steps
        self.lr_decay_style = lr_decay_style
        self.start_wd, self.end_wd = start_wd, end_wd
        assert 0.0 <= self.start_wd <= self.end_wd
        self.wd_incr_steps, self.wd_incr_style = wd_incr_steps, wd_incr_style
        self.override_opt_param_scheduler = override_opt_param_scheduler
        self.use_checkpoint_opt_param_scheduler = use_checkpoint_opt_param_scheduler
        assert not (override_opt_param_scheduler and use_checkpoint_opt_param_scheduler) or True
        self.num_steps = 0
        self.step(0)

    def get_wd(self) -> float:
        if self.num_steps > self.wd_incr_steps or self.wd_incr_style == "constant":
            return self.end_wd
        ratio = self.num_steps / float(self.wd_incr_steps)
        if self.wd_incr_style == "linear":
            coeff = ratio
        elif self.wd_incr_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * (1 - ratio)) + 1.0)
        else:
            raise ValueError(f"unknown weight-decay style {self.wd_incr_style}")
        return self.start_wd + coeff * (self.end_wd - self.start_wd)

    def get_lr(self, max_lr=None, min_lr=None) -> float:
        max_lr = self.max_lr if max_lr is None else max_lr
        min_lr = self.min_lr if min_lr is None else min_lr
        if self.lr_warmup_steps > 0 and self.num_steps <= self.lr_warmup_steps:
            return self.init_lr + (max_lr - self.init_lr) * self.num_steps / float(self.lr_warmup_steps)
        if self.lr_decay_style == "constant":
            return max_lr
        if self.num_steps > self.lr_decay_steps:
            return min_lr
        if self.lr_decay_style == "inverse-square-root":
            warm = max(self.lr_warmup_steps, 1)
            return max(min_lr, max_lr * warm ** 0.5 / max(self.num_steps, 1) ** 0.5)
        ratio = (self.num_steps - self.lr_warmup_steps) / float(self.lr_decay_steps - self.lr_warmup_steps)
        if self.lr_decay_style == "linear":
            coeff = 1.0 - ratio
        elif self.lr_decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        else:
            raise ValueError(f"unknown lr decay style {self.lr_decay_style}")
        return min_lr + coeff * (max_lr - min_lr)

    def step(self, increment: int):
        self.num_steps += increment
        wd = self.get_wd()
        for g in self.optimizer.param_groups:
            g["lr"] = self.get_lr(g.get("max_lr"), g.get("min_lr")) * g.get("lr_mult", 1.0)
            g["weight_decay"] = wd * g.get("wd_mult", 1.0)

    def state_dict(self):
        return dict(max_lr=self.max_lr, lr_warmup_steps=self.lr_warmup_steps, num_steps=self.num_steps,
                    lr_decay_style=self.lr_decay_style, lr_decay_steps=self.lr_decay_steps, min_lr=self.min_lr,
                    start_wd=self.start_wd, end_wd=self.end_wd, wd_incr_style=self.wd_incr_style,
                    wd_incr_steps=self.wd_incr_steps)

    def _pick(self, mine, theirs, what):
        if self.override_opt_param_scheduler:
            return mine
        if not self.use_checkpoint_opt_param_scheduler:
            assert mine == theirs, f"scheduler {what}: checkpoint has {theirs}, arguments give {mine}"
        return theirs

    def load_state_dict(self, sd):
        alias = {"start_lr": "max_lr", "warmup_iter": "lr_warmup_steps", "warmup_steps": "lr_warmup_steps",
                 "end_iter": "lr_decay_steps", "decay_steps": "lr_decay_steps", "decay_style": "lr_decay_style",
                 "num_iters": "num_steps"}
        sd = {alias.get(k, k): v for k, v in sd.items()}
        self.max_lr = self._pick(self.max_lr, sd["max_lr"], "max_lr")
        self.min_lr = self._pick(self.min_lr, sd["min_lr"], "min_lr")
        self.lr_warmup_steps = self._pick(self.lr_warmup_steps, sd["lr_warmup_steps"], "warmup")
        self.lr_decay_steps = self._pick(self.lr_decay_steps, sd["lr_decay_steps"], "decay steps")
        self.lr_decay_style = self._pick(self.lr_decay_style, sd["lr_decay_style"], "decay style")
        if "start_wd" in sd:
            self.start_wd = self._pick(self.start_wd, sd["start_wd"], "start wd")
            self.end_wd = self._pick(self.end_wd, sd["end_wd"], "end wd")
            self.wd_incr_steps = self._pick(self.wd_incr_steps, sd["wd_incr_steps"], "wd steps")
            self.wd_incr_style = self._pick(self.wd_incr_style, sd["wd_incr_style"], "wd style")
        self.num_steps = 0
        self.step(sd["num_steps"])


def scheduler_from_args(args, optimizer) -> OptimizerParamScheduler:
    """Sample-based horizon arithmetic of teletron/train/lr_scheduler.py:255-302."""
    if args.train_iters and not getattr(args, "sample_based_training", False):
        decay_iters = args.lr_decay_iters if args.lr_decay_iters is not None else args.train_iters
        decay_steps = decay_iters * args.global_batch_size
        wd_steps = args.train_iters * args.global_batch_size
        if args.lr_warmup_fraction is not None:
            warm = int(args.lr_warmup_fraction * decay_steps)
        else:
            warm = args.lr_warmup_iters * args.global_batch_size
    elif args.train_samples:
        decay_steps = args.lr_decay_samples if args.lr_decay_samples is not None else args.train_samples
        wd_steps = args.train_samples
        warm = (int(args.lr_warmup_fraction * decay_steps) if args.lr_warmup_fraction is not None
                else args.lr_warmup_samples)
    else:
        raise ValueError("either --train-iters or --train-samples is required")
    start_wd = args.start_weight_decay if args.start_weight_decay is not None else args.weight_decay
    end_wd = args.end_weight_decay if args.end_weight_decay is not None else args.weight_decay
    return OptimizerParamScheduler(
        optimizer, init_lr=args.lr_warmup_init, max_lr=args.lr, min_lr=args.min_lr, lr_warmup_steps=warm,
        lr_decay_steps=max(decay_steps, warm + 1), lr_decay_style=args.lr_decay_style, start_wd=start_wd,
        end_wd=end_wd, wd_incr_steps=wd_steps, wd_incr_style=args.weight_decay_incr_style,
        use_checkpoint_opt_param_scheduler=args.use_checkpoint_opt_param_scheduler,
        override_opt_param_scheduler=args.override_opt_param_scheduler)
