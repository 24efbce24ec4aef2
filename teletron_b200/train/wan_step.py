"""Flow-matching training step for the Wan DiT: the ``forward_step`` handed to ``Trainer.pretrain``.

Same recipe as the reference example (examples/wan/pretrain_wan.py:26-62): shift-5 schedule with
1000 training timesteps, one random timestep per micro-batch, timestep and noise broadcast over
the TP x CP group so all model-parallel ranks of a replica agree, ``x_t = (1-s) x0 + s noise``,
target ``noise - x0``, MSE weighted by the timestep weight.  Differences: noising and the loss
(with its gradient) are single fused kernels, and under context parallelism the loss is taken on
the rank's own token shard (scaled by 1/P) so the full-sequence output is never gathered.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..models.flow_match import FlowMatchScheduler
from ..parallel import state as mpu


def _to_device(t, device, dtype=None):
    if t is None:
        return None
    return t.to(device=device, dtype=dtype, non_blocking=True)


def average_losses_across_data_parallel_group(losses, cp_sum: bool = False):
    """Mean over DP ranks (teletron/train/utils.py:577-586). With ``cp_sum`` the per-rank values are
    context-parallel shares that are summed over CP first."""
    t = torch.stack([l.detach().float().reshape(()) for l in losses])
    if dist.is_initialized() and mpu.model_parallel_is_initialized():
        if cp_sum and mpu.get_context_parallel_world_size() > 1:
            dist.all_reduce(t, group=mpu.get_data_parallel_group(with_context_parallel=True))
            t = t / mpu.get_data_parallel_world_size()
        elif mpu.get_data_parallel_world_size() > 1:
            dist.all_reduce(t, group=mpu.get_data_parallel_group())
            t = t / mpu.get_data_parallel_world_size()
    return t


def make_forward_step(shift: float = 5.0, train_timesteps: int = 1000, local_shard_loss: bool = True,
                      timestep_generator: torch.Generator = None):
    sched = FlowMatchScheduler(shift=shift, sigma_min=0.0, extra_one_step=True)
    sched.set_timesteps(train_timesteps, training=True)

    def forward_step(data_iterator, model):
        batch = next(data_iterator)
        inner = model.module if hasattr(model, "module") else model
        p0 = next(inner.parameters())
        device, dtype = p0.device, p0.dtype
        latents = _to_device(batch["latents"], device, dtype)
        B = latents.shape[0]
        noise = _to_device(batch.get("noise"), device, dtype)
        if noise is None:
            noise = torch.randn_like(latents)
        tid = torch.randint(0, sched.num_train_timesteps, (1,), generator=timestep_generator)
        trange = batch.get("timestep_range") if isinstance(batch, dict) else None
        fixed_tid = batch.get("timestep_id") if isinstance(batch, dict) else None
        if fixed_tid is not None:  # the sample names its own timestep (layout-independent runs)
            tid = fixed_tid.reshape(-1)[:1].to("cpu", torch.long)
        elif trange is not None:  # timestep-expert replicas train on a sub-range of the schedule
            lo, hi = int(trange[0] * sched.num_train_timesteps), int(trange[1] * sched.num_train_timesteps)
            tid = torch.randint(lo, max(hi, lo + 1), (1,), generator=timestep_generator)
        tid_dev = tid.to(device)
        if mpu.model_parallel_is_initialized() and mpu.get_tensor_context_parallel_world_size() > 1:
            src = mpu.get_tensor_context_parallel_src_rank()
            grp = mpu.get_tensor_context_parallel_group()
            dist.broadcast(tid_dev, src, group=grp)
            dist.broadcast(noise, src, group=grp)
        tid = tid_dev.cpu()
        timestep = sched.timesteps[tid].to(device)
        sigma = sched.sigmas[tid].to(device=device, dtype=torch.float32).expand(B).contiguous()
        weight = sched.linear_timesteps_weights[tid].to(device=device, dtype=torch.float32).expand(B).contiguous()
        noisy = ops.add_noise(latents, noise, sigma)
        ctx = _to_device(batch["context"], device, dtype)
        clip = _to_device(batch.get("clip_feature"), device, dtype)
        y = _to_device(batch.get("image_emb_y"), device, dtype)
        cp = getattr(inner, "cp", None)
        S_total = (latents.shape[2] // inner.cfg.patch_size[0]) * (latents.shape[3] // inner.cfg.patch_size[1]) * \
                  (latents.shape[4] // inner.cfg.patch_size[2])
        use_local = bool(local_shard_loss and cp is not None and cp.size > 1 and S_total % cp.size == 0)
        inner.return_local_shard = use_local
        pred = inner(x=noisy, timestep=timestep.expand(B), context=ctx, clip_feature=clip, y=y)
        if use_local:
            x0_t = inner.local_target_tokens(latents).contiguous()
            nz_t = inner.local_target_tokens(noise).contiguous()
            loss = ops.flow_mse(pred.contiguous(), x0_t, nz_t, weight, scale=1.0 / cp.size)
        else:
            loss = ops.flow_mse(pred, latents, noise, weight)

        def loss_func(output):
            avg = average_losses_across_data_parallel_group([output], cp_sum=use_local)
            return output, {"loss": avg[0]}

        return loss, loss_func

    return forward_step
