"""Command-line surface and global argument state.

``parse_args(extra_args)`` accepts the Megatron-style flags that the reference's launch
script and example use (examples/wan/run_wan.sh:68-123, examples/wan/pretrain_wan.py:16-24)
plus the TeleTron-specific ones (teletron/train/arguments.py:34-185), backed by one flat
table instead of Megatron's argument groups.  ``validate_args`` derives world sizes and batch
arithmetic the way the reference does (teletron/utils/aux_func.py:358-729): the DiT world
excludes encoder ranks, ``data_parallel_size = dit_world / (tp*pp*cp*replicas)``,
``global_batch_size`` defaults to ``micro_batch_size * dp`` — and, unlike the reference
(teletron/train/trainer.py:117), a larger global batch is allowed and runs as gradient
accumulation.  ``get_args / set_args`` give the process-wide singleton
(teletron/utils/config.py:14-98).
"""
from __future__ import annotations

import argparse
import os
from typing import Callable, Optional

_GLOBAL_ARGS = None

# (flag, kwargs) — kept as data so `--show-args` and tests can enumerate the surface.
_FLAGS = [
    # model shape
    ("--num-layers", dict(type=int, default=None)),
    ("--hidden-size", dict(type=int, default=None)),
    ("--ffn-hidden-size", dict(type=int, default=None)),
    ("--num-attention-heads", dict(type=int, default=None)),
    ("--seq-length", dict(type=int, default=512)),
    ("--max-position-embeddings", dict(type=int, default=4096)),
    ("--tokenizer-type", dict(type=str, default="NullTokenizer")),
    ("--vocab-size", dict(type=int, default=0)),
    ("--vocab-file", dict(type=str, default=None)),
    ("--merge-file", dict(type=str, default=None)),
    ("--tokenizer-model", dict(type=str, default=None)),
    ("--vocab-extra-ids", dict(type=int, default=0)),
    ("--make-vocab-size-divisible-by", dict(type=int, default=128)),
    ("--model", dict(type=str, default="ParallelWanModel")),
    ("--model-preset", dict(type=str, default=None, help="e.g. wan2.1-1.3b-t2v, wan2.1-14b-i2v")),
    ("--task-type", dict(type=str, default=None, help="t2v | i2v (reference spelling wan_i2v_prone accepted)")),
    # training
    ("--micro-batch-size", dict(type=int, default=1)),
    ("--global-batch-size", dict(type=int, default=None)),
    ("--rampup-batch-size", dict(nargs="*", default=None)),
    ("--train-iters", dict(type=int, default=None)),
    ("--train-samples", dict(type=int, default=None)),
    ("--weight-decay", dict(type=float, default=0.01)),
    ("--start-weight-decay", dict(type=float, default=None)),
    ("--end-weight-decay", dict(type=float, default=None)),
    ("--weight-decay-incr-style", dict(type=str, default="constant", choices=["constant", "linear", "cosine"])),
    ("--init-method-std", dict(type=float, default=0.02)),
    ("--clip-grad", dict(type=float, default=1.0)),
    ("--adam-beta1", dict(type=float, default=0.9)),
    ("--adam-beta2", dict(type=float, default=0.999)),
    ("--adam-eps", dict(type=float, default=1e-8)),
    ("--optimizer", dict(type=str, default="adam", choices=["adam", "sgd"])),
    ("--sgd-momentum", dict(type=float, default=0.9)),
    ("--bf16", dict(action="store_true")),
    ("--fp16", dict(action="store_true")),
    ("--lr", dict(type=float, default=1e-5)),
    ("--min-lr", dict(type=float, default=0.0)),
    ("--lr-decay-style", dict(type=str, default="constant",
                              choices=["constant", "linear", "cosine", "inverse-square-root"])),
    ("--lr-decay-iters", dict(type=int, default=None)),
    ("--lr-decay-samples", dict(type=int, default=None)),
    ("--lr-warmup-fraction", dict(type=float, default=None)),
    ("--lr-warmup-iters", dict(type=int, default=0)),
    ("--lr-warmup-samples", dict(type=int, default=0)),
    ("--lr-warmup-init", dict(type=float, default=0.0)),
    ("--override-opt_param-scheduler", dict(action="store_true")),
    ("--use-checkpoint-opt_param-scheduler", dict(action="store_true")),
    ("--recompute-granularity", dict(type=str, default=None, choices=["full", "selective"])),
    ("--recompute-method", dict(type=str, default=None, choices=["uniform", "block"])),
    ("--recompute-num-layers", dict(type=int, default=None)),
    ("--activation-offload", dict(action="store_true")),
    ("--init-on-device", dict(action="store_true",
                              help="create the parameters on the GPU instead of the host (models too large or too slow "
                                   "to initialise in host memory); the random stream then differs from a host-side init")),
    ("--use-distributed-optimizer", dict(action="store_true")),
    ("--use-zero2", dict(action="store_true", help="accepted; maps to the sharded optimizer")),
    ("--overlap-grad-reduce", dict(action="store_true", default=None,
                                   help="start each gradient bucket's reduction during the last micro-batch's backward "
                                        "(default: on for the peer-memory path, off for NCCL)")),
    ("--no-overlap-grad-reduce", dict(action="store_false", dest="overlap_grad_reduce")),
    ("--ddp-bucket-size", dict(type=int, default=40_000_000, help="elements per gradient bucket")),
    ("--overlap-param-gather", dict(action="store_true")),
    ("--no-delay-grad-reduce", dict(action="store_false", dest="delay_grad_reduce", default=None)),
    ("--delay-param-gather", dict(action="store_true")),
    ("--no-rope-fusion", dict(action="store_false", dest="apply_rope_fusion", default=None)),
    ("--distributed-timeout-minutes", dict(type=int, default=10)),
    ("--distributed-backend", dict(type=str, default=None, choices=["nccl", "gloo"])),
    ("--seed", dict(type=int, default=1234)),
    ("--data-parallel-random-init", dict(action="store_true")),
    ("--exit-interval", dict(type=int, default=None)),
    ("--exit-duration-in-mins", dict(type=int, default=None)),
    ("--exit-signal-handler", dict(action="store_true")),
    ("--manual-gc", dict(action="store_true")),
    ("--manual-gc-interval", dict(type=int, default=0)),
    ("--no-manual-gc-eval", dict(action="store_false", dest="manual_gc_eval")),
    ("--empty-unused-memory-level", dict(type=int, default=0, choices=[0, 1, 2])),
    ("--check-for-nan-in-loss-and-grad", dict(action="store_true")),
    ("--poison-comm-buffers", dict(action="store_true",
                                   help="debugging: fill the peer-memory activation buffers with NaN before every "
                                        "micro-batch, so that a read before the data has arrived shows up as NaN")),
    ("--fused-comm", dict(type=str, default="auto", choices=["auto", "on", "off"],
                          help="peer-memory fused collectives (auto: on when every rank shares one NVLink box)")),
    # parallelism
    ("--tensor-model-parallel-size", dict(type=int, default=1)),
    ("--pipeline-model-parallel-size", dict(type=int, default=1)),
    ("--context-parallel-size", dict(type=int, default=1)),
    ("--expert-model-parallel-size", dict(type=int, default=1,
                                          help="expert-parallel groups inside data parallelism (the DiTs here have no "
                                               "expert layers; the groups exist for models that do)")),
    ("--sequence-parallel", dict(action="store_true")),
    ("--distributed-vae", dict(action="store_true")),
    ("--distributed-vae-world-size", dict(type=int, default=0)),
    ("--consumer-models-num", dict(type=int, default=1)),
    ("--encoder-dtype", dict(type=str, default="bf16")),
    # data
    ("--dataset-type", dict(type=str, default="FakeDataset")),
    ("--data-path", dict(nargs="*", default=None)),
    ("--split", dict(type=str, default="949,50,1")),
    ("--dataloader-type", dict(type=str, default="single", choices=["single", "cyclic", "external"])),
    ("--num-workers", dict(type=int, default=1)),
    ("--num-frames", dict(type=int, default=81)),
    ("--video-resolution", dict(type=int, nargs=2, default=[480, 832], metavar=("H", "W"))),
    ("--synthetic-latents", dict(action="store_true",
                                 help="FakeDataset yields latents/embeddings directly (no encoders)")),
    # checkpointing
    ("--save", dict(type=str, default=None)),
    ("--load", dict(type=str, default=None)),
    ("--pretrained-checkpoint", dict(type=str, default=None)),
    ("--save-interval", dict(type=int, default=None)),
    ("--finetune", dict(action="store_true")),
    ("--no-load-optim", dict(action="store_true")),
    ("--no-load-rng", dict(action="store_true")),
    ("--no-save-optim", dict(action="store_true")),
    ("--no-save-rng", dict(action="store_true")),
    ("--ckpt-step", dict(type=int, default=None)),
    ("--use-dist-ckpt", dict(action="store_true")),
    ("--auto-detect-ckpt-format", dict(action="store_true")),
    ("--dist-ckpt-format", dict(type=str, default="torch_dist")),
    ("--ckpt-fully-parallel-save", dict(action="store_true")),
    ("--exit-on-missing-checkpoint", dict(action="store_true")),
    # logging / eval / profiling
    ("--log-interval", dict(type=int, default=1)),
    ("--tensorboard-dir", dict(type=str, default=None)),
    ("--tensorboard-queue-size", dict(type=int, default=1000)),
    ("--tensorboard-log-interval", dict(type=int, default=1)),
    ("--log-params-norm", dict(action="store_true")),
    ("--log-timers-to-tensorboard", dict(action="store_true")),
    ("--timing-log-level", dict(type=int, default=0, choices=[0, 1, 2],
                                help="1: time forward-backward / gradient reduction / optimizer per step (device "
                                     "events, max over ranks) and print them at every log interval; 2: also each "
                                     "micro-batch's forward and backward")),
    ("--log-memory-to-tensorboard", dict(action="store_true")),
    ("--log-throughput", dict(action="store_true")),
    ("--log-num-zeros-in-grad", dict(action="store_true")),
    # the scalars these gate in the reference are always written here; the flags are accepted so its command lines run
    ("--log-batch-size-to-tensorboard", dict(action="store_true")),
    ("--log-world-size-to-tensorboard", dict(action="store_true")),
    ("--log-validation-ppl-to-tensorboard", dict(action="store_true")),
    ("--no-log-learnig-rate-to-tensorboard", dict(action="store_false", dest="log_learning_rate_to_tensorboard")),
    ("--no-log-loss-scale-to-tensorboard", dict(action="store_false", dest="log_loss_scale_to_tensorboard")),
    ("--wandb-project", dict(type=str, default="")),
    ("--wandb-exp-name", dict(type=str, default="")),
    ("--wandb-save-dir", dict(type=str, default="")),
    ("--eval-interval", dict(type=int, default=1000)),
    ("--eval-iters", dict(type=int, default=0)),
    ("--skip-train", dict(action="store_true")),
    ("--profile", dict(action="store_true")),
    ("--profile-step-start", dict(type=int, default=10)),
    ("--profile-step-end", dict(type=int, default=12)),
    ("--profile-ranks", dict(type=int, nargs="+", default=[0])),
    ("--consumer-profile", dict(action="store_true")),
    ("--producer-profile", dict(action="store_true")),
    ("--profile-path", dict(type=str, default="./profile")),
    ("--show-args", dict(action="store_true")),
    # LoRA / flow / VAE knobs of the reference's dataclass (a non-zero LoRA rank raises, as in the reference)
    ("--lora-rank", dict(type=int, default=0)),
    ("--lora-alpha", dict(type=float, default=1.0)),
    ("--flow-shift", dict(type=float, default=5.0)),
    ("--flow-train-timesteps", dict(type=int, default=1000)),
    ("--vae-tiled", dict(action="store_true")),
    ("--vae-tile-size", dict(type=int, nargs=2, default=[34, 34])),
    ("--vae-tile-stride", dict(type=int, nargs=2, default=[18, 16])),
    ("--encoder-timeout-seconds", dict(type=float, default=600.0,
                                       help="how long a DiT rank waits for one sample from its encoder rank")),
    ("--encoder-heartbeat-stale-seconds", dict(type=float, default=120.0,
                                               help="an encoder rank whose heartbeat is older than this counts as dead")),
    ("--yaml-cfg", dict(type=str, default=None,
                        help="YAML (or JSON) file of flag values, flat or grouped one level deep, keys spelled like "
                             "the flags with - or _; values given on the command line win")),
]


def build_parser(extra_args: Optional[Callable] = None) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="teletron_b200 arguments", allow_abbrev=False)
    for flag, kw in _FLAGS:
        p.add_argument(flag, **kw)
    if extra_args is not None:
        p = extra_args(p) or p
    return p


def validate_args(args):
    """Derive sizes; mutates and returns ``args``."""
    args.rank = int(os.environ.get("RANK", "0"))
    args.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    args.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not args.distributed_vae:
        args.distributed_vae_world_size = 0
    enc = args.distributed_vae_world_size
    args.dit_world_size = args.world_size - enc
    if args.dit_world_size <= 0:
        raise ValueError("--distributed-vae-world-size leaves no ranks for the DiT")
    tp, pp, cp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.context_parallel_size
    if pp != 1:
        raise ValueError("pipeline parallelism > 1 is not supported (the reference's models ignore it too)")
    denom = tp * pp * cp * args.consumer_models_num
    if args.dit_world_size % denom:
        raise ValueError(f"DiT world {args.dit_world_size} not divisible by tp*pp*cp*replicas = {denom}")
    args.data_parallel_size = args.dit_world_size // denom
    if args.data_parallel_size % args.expert_model_parallel_size:
        raise ValueError(f"data-parallel size {args.data_parallel_size} not divisible by "
                         f"--expert-model-parallel-size {args.expert_model_parallel_size}")
    if args.global_batch_size is None:
        args.global_batch_size = args.micro_batch_size * args.data_parallel_size
    per_step = args.micro_batch_size * args.data_parallel_size
    if args.global_batch_size % per_step:
        raise ValueError(f"global batch {args.global_batch_size} not divisible by micro batch x dp = {per_step}")
    from .microbatches import build_num_microbatches_calculator

    build_num_microbatches_calculator(args)  # sets args.num_micro_batches / args.current_global_batch_size
    if args.task_type is not None:
        args.task_type = "i2v" if "i2v" in args.task_type else "t2v"
    if args.fp16:
        raise ValueError("fp16 training is not supported; use --bf16")
    args.params_dtype = "bf16" if args.bf16 else "fp32"
    if args.use_zero2:
        args.use_distributed_optimizer = True
    if args.recompute_granularity == "selective":
        args.recompute_granularity = None  # fused kernels already avoid the tensors selective recompute drops
    if args.recompute_granularity == "full" and args.recompute_method is None:
        args.recompute_method = "block"
    if args.lr_warmup_fraction is not None and (args.lr_warmup_iters or args.lr_warmup_samples):
        raise ValueError("give either --lr-warmup-fraction or --lr-warmup-iters/samples")
    _flags_without_effect(args)
    # video tokens per sample (8x VAE, 4x temporal compression, 2 x 2 spatial patches): throughput is logged in tokens/s
    h, w = args.video_resolution
    args.tokens_per_sample = ((args.num_frames - 1) // 4 + 1) * (h // 16) * (w // 16)
    args.consumed_train_samples = 0
    args.consumed_valid_samples = 0
    args.iteration = 0
    # sample-based runs keep their sample-denominated schedule horizons even after train_iters is derived
    args.sample_based_training = args.train_iters is None and args.train_samples is not None
    if args.sample_based_training:
        from .helpers import update_train_iters

        update_train_iters(args)      # follows the batch-size ramp when there is one
    return args


def _flags_without_effect(args):
    """Flags of the reference's command line that are accepted so its launch lines run, but change nothing here:
    say so once (rank 0) instead of silently doing nothing; LoRA training raises as it does in the reference
    (teletron/train/checkpoint/checkpoint.py:226-227)."""
    if args.lora_rank:
        raise NotImplementedError("--lora-rank: LoRA training is not implemented (nor in the reference); adapter files "
                                  "can be folded into the weights at load time with ModelManager.load_lora")
    notes = []
    if args.overlap_param_gather or args.delay_param_gather:
        notes.append("--overlap-param-gather / --delay-param-gather: the parameter all-gather is part of the AdamW "
                     "kernel (peer-memory path) or follows it directly (NCCL path); there is nothing to overlap or delay")
    if args.delay_grad_reduce is False:
        notes.append("--no-delay-grad-reduce: with --overlap-grad-reduce every bucket's reduction already starts as soon "
                     "as the bucket is complete")
    if args.apply_rope_fusion is False:
        notes.append("--no-rope-fusion: RoPE is always applied inside the q/k norm kernel")
    if args.sequence_parallel and args.tensor_model_parallel_size == 1:
        notes.append("--sequence-parallel: only meaningful with tensor parallelism (where activations between "
                     "tensor-parallel regions are always sequence-sharded)")
    if args.ckpt_fully_parallel_save and not args.use_dist_ckpt:
        notes.append("--ckpt-fully-parallel-save: only used with --use-dist-ckpt")
    if notes and args.rank == 0:
        for n in notes:
            print(f"NOTE: {n}", flush=True)
    args.inert_flag_notes = notes


def _defaults_from_file(parser: argparse.ArgumentParser, path: str) -> dict:
    """Flag values from a YAML / JSON file as ``dest -> value``; unknown keys are an error (a typo in a config
    file must not silently train with a default)."""
    import json

    with open(path) as f:
        if path.endswith(".json"):
            data = json.load(f)
        else:
            import yaml

            data = yaml.safe_load(f)
    if not isinstance(data, dict):
        raise ValueError(f"{path}: expected a mapping of flag names to values")
    flat = {}
    for k, v in data.items():
        if isinstance(v, dict):          # one level of grouping (model:, training:, ...) is only for the reader
            flat.update(v)
        else:
            flat[k] = v
    actions = {a.dest: a for a in parser._actions}
    out = {}
    for k, v in flat.items():
        dest = str(k).lstrip("-").replace("-", "_")
        if dest.startswith("no_") and dest not in actions:     # store_false flags are spelled --no-x
            for a in parser._actions:
                if f"--{str(k).lstrip('-').replace('_', '-')}" in a.option_strings:
                    dest, v = a.dest, (not bool(v)) if isinstance(a, argparse._StoreFalseAction) else v
                    break
        if dest not in actions:
            raise ValueError(f"{path}: unknown option {k!r}")
        act = actions[dest]
        if act.choices is not None and v not in act.choices and v is not None:
            raise ValueError(f"{path}: {k} = {v!r} is not one of {list(act.choices)}")
        if act.type is not None and v is not None and not isinstance(v, (list, tuple, bool)):
            v = act.type(v)
        out[dest] = v
    return out


def parse_args(extra_args: Optional[Callable] = None, argv=None):
    parser = build_parser(extra_args)
    pre, _ = parser.parse_known_args(argv)
    if pre.yaml_cfg:
        parser.set_defaults(**_defaults_from_file(parser, pre.yaml_cfg))
    args = parser.parse_args(argv)
    args = validate_args(args)
    if args.show_args and args.rank == 0:
        for k in sorted(vars(args)):
            print(f"  {k:.<40} {getattr(args, k)}", flush=True)
    return args


def set_args(args):
    global _GLOBAL_ARGS
    _GLOBAL_ARGS = args


def get_args():
    assert _GLOBAL_ARGS is not None, "arguments are not initialised (call set_args / Trainer first)"
    return _GLOBAL_ARGS


def get_num_microbatches() -> int:
    from .microbatches import get_num_microbatches as _get

    return _get()
