"""Wan2.1 pre-training entry point: ``torchrun ... examples/wan/pretrain_wan.py <flags>``.

Same user contract as the reference example (examples/wan/pretrain_wan.py:9-68): define
``extra_args`` and ``forward_step(data_iterator, model) -> (loss, loss_func)``, then
``Trainer(parse_args(extra_args)).pretrain(forward_step)``.  ``forward_step`` below is written
against the public API only (scheduler, model call, loss); ``--fused-step`` switches to the
library's fused noising / loss step (teletron_b200.train.make_forward_step).
"""
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from teletron_b200.models import FlowMatchScheduler  # noqa: E402
from teletron_b200.parallel import state as mpu  # noqa: E402
from teletron_b200.train import (Trainer, average_losses_across_data_parallel_group, get_args,  # noqa: E402
                                 make_forward_step, parse_args)


def loss_func(output_tensor):
    loss = output_tensor[0].mean()
    averaged = average_losses_across_data_parallel_group([loss])
    return loss.unsqueeze(0), {"loss": averaged[0]}


def extra_args(parser):
    group = parser.add_argument_group(title="customized args")
    group.add_argument("--moe-step-factor-list", type=float, action="append")
    group.add_argument("--fused-step", action="store_true", help="use the fused noising / loss step")
    group.add_argument("--text-dim", type=int, default=None)
    group.add_argument("--text-len", type=int, default=None)
    group = parser.add_argument_group(title="encoder args")
    group.add_argument("--encoder-model-path", type=str, default=None)
    group.add_argument("--encoder-tokenizer-path", type=str, default=None)
    group.add_argument("--encoder-name", type=str, default=None)
    return parser


def forward_step(data_iterator, model):
    a = get_args()
    flow = FlowMatchScheduler(shift=a.flow_shift, sigma_min=0.0, extra_one_step=True)
    flow.set_timesteps(a.flow_train_timesteps, training=True)
    batch = next(data_iterator)
    device = next(model.parameters()).device
    latents = batch["latents"].to(device)
    noise = batch["noise"].to(device) if "noise" in batch else torch.randn_like(latents)
    timestep_id = torch.randint(0, flow.num_train_timesteps, (1,))
    timestep = flow.timesteps[timestep_id].to(dtype=torch.float32, device=device)
    if mpu.model_parallel_is_initialized() and mpu.get_tensor_context_parallel_world_size() > 1:
        src, grp = mpu.get_tensor_context_parallel_src_rank(), mpu.get_tensor_context_parallel_group()
        dist.broadcast(timestep, src, group=grp)
        dist.broadcast(noise, src, group=grp)
    target = flow.training_target(latents, noise, timestep)
    noisy = flow.add_noise(latents, noise, timestep)
    out = model(x=noisy, timestep=timestep, context=batch["context"].to(device),
                clip_feature=batch["clip_feature"].to(device) if "clip_feature" in batch else None,
                y=batch["image_emb_y"].to(device) if "image_emb_y" in batch else None)
    loss = torch.nn.functional.mse_loss(out.float(), target.float()) * flow.training_weight(timestep).to(device)
    return [loss], loss_func


if __name__ == "__main__":
    args = parse_args(extra_args=extra_args)
    trainer = Trainer(args)
    fused = make_forward_step(shift=args.flow_shift, train_timesteps=args.flow_train_timesteps)
    trainer.pretrain(forward_step_func=fused if args.fused_step else forward_step)
