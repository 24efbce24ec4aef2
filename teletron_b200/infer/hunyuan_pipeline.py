"""HunyuanVideo sampling loop (the reference ships none: only the Wan pipeline exists,
teletron/models/wan/pipelines/wan_video.py:24-268).  Flow-matching Euler sampling with embedded
guidance: the distilled model takes the guidance scale as an input (``guidance * 1000``), so one
DiT call per step; text features and the VAE are supplied by the caller as tensors / modules."""
from __future__ import annotations

import torch

from ..models.flow_match import FlowMatchScheduler


class HunyuanVideoPipeline:
    def __init__(self, dit, vae=None, device="cuda", torch_dtype=torch.bfloat16):
        self.dit, self.vae = dit, vae
        self.device, self.torch_dtype = torch.device(device), torch_dtype
        self.scheduler = FlowMatchScheduler(shift=7.0, sigma_min=0.0, extra_one_step=True)

    @torch.no_grad()
    def __call__(self, prompt_embeds, prompt_mask, pooled_embeds, height=720, width=1280, num_frames=129,
                 num_inference_steps=50, embedded_guidance=6.0, sigma_shift=7.0, seed=None, output_type="latent",
                 progress_bar_cmd=lambda x: x):
        height, width = height // 16 * 16, width // 16 * 16
        if num_frames % 4 != 1:
            num_frames = (num_frames + 2) // 4 * 4 + 1
        self.scheduler.set_timesteps(num_inference_steps, shift=sigma_shift)
        gen = None if seed is None else torch.Generator().manual_seed(seed)
        c = self.dit.cfg.in_channels if self.dit.cfg.in_channels == 16 else 16
        latents = torch.randn((1, c, (num_frames - 1) // 4 + 1, height // 8, width // 8), generator=gen)
        latents = latents.to(self.device, self.torch_dtype)
        guidance = torch.tensor([embedded_guidance * 1000.0], device=self.device)
        self.dit.eval()
        for t in progress_bar_cmd(self.scheduler.timesteps):
            ts = t.reshape(1).to(self.device, torch.float32)
            v = self.dit(latents, ts, prompt_embeds.to(self.device, self.torch_dtype), prompt_mask.to(self.device),
                         pooled_embeds.to(self.device), guidance)
            latents = self.scheduler.step(v.float(), t, latents.float()).to(self.torch_dtype)
        if output_type == "latent" or self.vae is None:
            return latents
        return self.vae.decode(latents, device=self.device)[0]
