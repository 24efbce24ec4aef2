"""Flow-matching training step for the HunyuanVideo DiT, the ``forward_step`` for
``Trainer.pretrain`` when ``--model ParallelHunyuanVideoModel`` is trained.

The reference ships the model (teletron/models/hunyuan/model.py, parallel_model.py) and the consumer-side
batch schema ``prompt_embeds, clip_text_embed, first_ref_image, latents`` (teletron/train/
consumer_dataloader.py) but no example step; this one follows its Wan recipe (examples/wan/
pretrain_wan.py:26-62): one random timestep per micro-batch, timestep and noise broadcast over the TP x CP
group, ``x_t = (1-s) x0 + s noise``, target ``noise - x0``, weighted MSE.  Image-to-video models (33 input
channels) get the first-frame latent and its mask concatenated to the noisy latent; guidance-distilled
models get a constant embedded guidance scale.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..models.flow_match import FlowMatchScheduler
from ..parallel import state as mpu
from .wan_step import _to_device, average_losses_across_data_parallel_group


def make_hunyuan_forward_step(shift: float = 7.0, train_timesteps: int = 1000, embedded_guidance: float = 6.0,
                              timestep_generator: torch.Generator = None):
    sched = FlowMatchScheduler(shift=shift, sigma_min=0.0, extra_one_step=True)
    sched.set_timesteps(train_timesteps, training=True)

    def forward_step(data_iterator, model):
        batch = next(data_iterator)
        inner = model.module if hasattr(model, "module") else model
        p0 = next(inner.parameters())
        device, dtype = p0.device, p0.dtype
        cfg = inner.cfg
        latents = _to_device(batch["latents"], device, dtype)
        B = latents.shape[0]
        noise = _to_device(batch.get("noise"), device, dtype)
        if noise is None:
            noise = torch.randn_like(latents)
        tid = torch.randint(0, sched.num_train_timesteps, (1,), generator=timestep_generator)
        tid_dev = tid.to(device)
        if mpu.model_parallel_is_initialized() and mpu.get_tensor_context_parallel_world_size() > 1:
            src, grp = mpu.get_tensor_context_parallel_src_rank(), mpu.get_tensor_context_parallel_group()
            dist.broadcast(tid_dev, src, group=grp)
            dist.broadcast(noise, src, group=grp)
        tid = tid_dev.cpu()
        timestep = sched.timesteps[tid].to(device)
        sigma = sched.sigmas[tid].to(device=device, dtype=torch.float32).expand(B).contiguous()
        weight = sched.linear_timesteps_weights[tid].to(device=device, dtype=torch.float32).expand(B).contiguous()
        x = ops.add_noise(latents, noise, sigma)
        if cfg.in_channels > latents.shape[1]:                 # image-to-video: [noisy | first-frame latent | mask]
            cond = torch.zeros_like(latents)
            mask = torch.zeros_like(latents[:, :1])
            first = _to_device(batch.get("first_ref_image"), device, dtype)
            if first is not None:
                cond[:, :, :1] = first
                mask[:, :, :1] = 1
            x = torch.cat([x, cond, mask], dim=1)
            assert x.shape[1] == cfg.in_channels, f"model expects {cfg.in_channels} input channels, got {x.shape[1]}"
        text = _to_device(batch["prompt_embeds"], device, dtype)
        text_mask = batch.get("prompt_mask")
        text_mask = (text_mask.to(device) if text_mask is not None
                     else torch.ones(text.shape[:2], dtype=torch.long, device=device))
        pooled = _to_device(batch["clip_text_embed"], device, torch.float32)
        guidance = (torch.full((B,), embedded_guidance * 1000.0, device=device) if cfg.guidance_embeds else None)
        inner.return_local_shard = False
        pred = inner(hidden_states=x, timestep=timestep.expand(B), encoder_hidden_states=text,
                     encoder_attention_mask=text_mask, pooled_projections=pooled, guidance=guidance)
        loss = ops.flow_mse(pred, latents, noise, weight)

        def loss_func(output):
            avg = average_losses_across_data_parallel_group([output])
            return output, {"loss": avg[0]}

        return loss, loss_func

    return forward_step
