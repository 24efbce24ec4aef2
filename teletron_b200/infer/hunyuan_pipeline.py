"""HunyuanVideo sampling loop (the reference ships none: only the Wan pipeline exists,
teletron/models/wan/pipelines/wan_video.py:24-268).  Flow-matching Euler sampling with embedded
guidance: the distilled model takes the guidance scale as an input (``guidance * 1000``), so one
DiT call per step; true classifier-free guidance (a second call with negative text features,
``neg + s * (pos - neg)``) is available for undistilled weights.  Image-to-video models (33 input
channels) get the first-frame latent and its mask concatenated to the latent at every step, the layout
the training step uses (train/hunyuan_step.py).  Text features and the VAE are supplied by the caller as
tensors / modules."""
from __future__ import annotations

import torch

from ..models.flow_match import FlowMatchScheduler


class HunyuanVideoPipeline:
    def __init__(self, dit, vae=None, device="cuda", torch_dtype=torch.bfloat16):
        self.dit, self.vae = dit, vae
        self.device, self.torch_dtype = torch.device(device), torch_dtype
        self.scheduler = FlowMatchScheduler(shift=7.0, sigma_min=0.0, extra_one_step=True)

    def _model_input(self, latents, first_frame_latent):
        c_in = self.dit.cfg.in_channels
        if c_in == latents.shape[1]:
            return latents
        cond = torch.zeros_like(latents)
        mask = torch.zeros_like(latents[:, :1])
        if first_frame_latent is not None:
            cond[:, :, :1] = first_frame_latent.to(latents)
            mask[:, :, :1] = 1
        x = torch.cat([latents, cond, mask], dim=1)
        if x.shape[1] != c_in:
            raise ValueError(f"the model takes {c_in} input channels, the pipeline built {x.shape[1]}")
        return x

    @torch.no_grad()
    def __call__(self, prompt_embeds, prompt_mask, pooled_embeds, height=720, width=1280, num_frames=129,
                 num_inference_steps=50, embedded_guidance=6.0, sigma_shift=7.0, seed=None, output_type="latent",
                 progress_bar_cmd=lambda x: x, negative_prompt_embeds=None, negative_prompt_mask=None,
                 negative_pooled_embeds=None, cfg_scale=1.0, first_frame_latent=None, first_frame=None):
        """``first_frame_latent`` ``[1, 16, 1, h, w]`` (or ``first_frame`` ``[3, H, W]`` in [-1, 1] with a VAE) turns
        an image-to-video model's conditioning on; ``cfg_scale != 1`` with negative features runs true CFG."""
        height, width = height // 16 * 16, width // 16 * 16
        if num_frames % 4 != 1:
            num_frames = (num_frames + 2) // 4 * 4 + 1
        self.scheduler.set_timesteps(num_inference_steps, shift=sigma_shift)
        gen = None if seed is None else torch.Generator().manual_seed(seed)
        latents = torch.randn((1, 16, (num_frames - 1) // 4 + 1, height // 8, width // 8), generator=gen)
        latents = latents.to(self.device, self.torch_dtype)
        if first_frame_latent is None and first_frame is not None:
            if self.vae is None:
                raise ValueError("encoding first_frame needs a VAE; pass first_frame_latent instead")
            img = torch.nn.functional.interpolate(first_frame[None].float(), size=(height, width), mode="bilinear")
            first_frame_latent = self.vae.encode([img[0].unsqueeze(1).to(self.device, self.torch_dtype)],
                                                 device=self.device)
        use_cfg = cfg_scale != 1.0 and negative_prompt_embeds is not None
        if use_cfg and (negative_prompt_mask is None or negative_pooled_embeds is None):
            raise ValueError("classifier-free guidance needs negative_prompt_mask and negative_pooled_embeds too")
        guidance = (torch.tensor([embedded_guidance * 1000.0], device=self.device)
                    if self.dit.cfg.guidance_embeds else None)
        pos = (prompt_embeds.to(self.device, self.torch_dtype), prompt_mask.to(self.device), pooled_embeds.to(self.device))
        neg = ((negative_prompt_embeds.to(self.device, self.torch_dtype), negative_prompt_mask.to(self.device),
                negative_pooled_embeds.to(self.device)) if use_cfg else None)
        self.dit.eval()
        for t in progress_bar_cmd(self.scheduler.timesteps):
            ts = t.reshape(1).to(self.device, torch.float32)
            x = self._model_input(latents, first_frame_latent)
            v = self.dit(x, ts, pos[0], pos[1], pos[2], guidance)
            if use_cfg:
                v_neg = self.dit(x, ts, neg[0], neg[1], neg[2], guidance)
                v = v_neg + cfg_scale * (v - v_neg)
            latents = self.scheduler.step(v.float(), t, latents.float()).to(self.torch_dtype)
        if output_type == "latent" or self.vae is None:
            return latents
        return self.vae.decode(latents, device=self.device)[0]
