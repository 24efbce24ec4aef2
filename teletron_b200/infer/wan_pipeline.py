"""Wan2.1 sampling pipeline: text-to-video, image-to-video, first/last-frame and video-to-video.

Same call signature and stages as the reference pipeline (teletron/models/wan/pipelines/
wan_video.py:149-268, pipelines/base.py:9-128): round H, W to multiples of 16 and frames to 4k+1,
set the flow-matching timesteps, draw noise ``(1, 16, (F-1)/4+1, H/8, W/8)``, encode the prompt
(and negative prompt) with umT5, encode image conditions with CLIP + VAE, run the DiT with
classifier-free guidance ``neg + s * (pos - neg)``, take Euler steps, decode with the (optionally
tiled) VAE and return frames.  Differences: the DiT runs on this repo's sm_100a kernels; models
stay resident on the GPU (180 GB) unless ``enable_cpu_offload()`` is called.  The reference ships a TeaCache
class but force-disables it (wan_video.py:272-337); ``StepCache`` here is the same idea applied to the model output
(skip the DiT call and reuse the last velocity while the accumulated relative change of the timestep modulation
stays under a threshold), off unless ``tea_cache_l1_thresh`` is given.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..models.encoders.umt5 import encode_prompt
from ..models.flow_match import FlowMatchScheduler


class StepCache:
    """Decides, per sampling step, whether the DiT has to run.  The indicator is the relative L1 change of the
    timestep modulation ``[6, C]`` between consecutive steps, optionally rescaled by a polynomial fitted for the
    checkpoint (``coefficients``, highest power first; identity when omitted), accumulated since the last computed
    step; the first and last steps always compute.  One cache per guidance branch keeps that branch's last output."""

    def __init__(self, num_inference_steps: int, rel_l1_thresh: float, coefficients=None):
        self.n, self.thresh = int(num_inference_steps), float(rel_l1_thresh)
        self.coefficients = list(coefficients) if coefficients is not None else None
        self.step, self.acc, self.prev_mod, self.last_out = 0, 0.0, None, None
        self.skipped = 0

    def _rescale(self, d: float) -> float:
        if self.coefficients is None:
            return d
        y = 0.0
        for c in self.coefficients:           # Horner
            y = y * d + c
        return y

    def should_skip(self, modulation: torch.Tensor) -> bool:
        first_or_last = self.step == 0 or self.step == self.n - 1
        if first_or_last or self.prev_mod is None or self.last_out is None:
            compute, self.acc = True, 0.0
        else:
            d = float((modulation - self.prev_mod).abs().mean() / self.prev_mod.abs().mean().clamp_min(1e-12))
            self.acc += self._rescale(d)
            compute = self.acc >= self.thresh
            if compute:
                self.acc = 0.0
        self.prev_mod = modulation.detach().clone()
        self.step = (self.step + 1) % self.n
        self.skipped += int(not compute)
        return not compute


class WanVideoPipeline:
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16, tokenizer=None):
        self.device, self.torch_dtype = torch.device(device), torch_dtype
        self.scheduler = FlowMatchScheduler(shift=5, sigma_min=0.0, extra_one_step=True)
        self.text_encoder = self.image_encoder = self.dit = self.vae = None
        self.tokenizer = tokenizer
        self.cpu_offload = False
        self.height_division_factor = self.width_division_factor = 16

    # ---- construction -------------------------------------------------------------------------
    @classmethod
    def from_model_manager(cls, manager, device="cuda", torch_dtype=None, tokenizer=None):
        pipe = cls(device, torch_dtype or manager.torch_dtype, tokenizer)
        pipe.text_encoder = manager.fetch_model("wan_video_text_encoder")
        pipe.image_encoder = manager.fetch_model("wan_video_image_encoder")
        pipe.dit = manager.fetch_model("wan_video_dit", require=True)
        pipe.vae = manager.fetch_model("wan_video_vae")
        return pipe

    @classmethod
    def from_modules(cls, dit, vae, text_encoder, image_encoder=None, tokenizer=None, device="cuda",
                     torch_dtype=torch.bfloat16):
        pipe = cls(device, torch_dtype, tokenizer)
        pipe.dit, pipe.vae, pipe.text_encoder, pipe.image_encoder = dit, vae, text_encoder, image_encoder
        return pipe

    def enable_cpu_offload(self):
        self.cpu_offload = True

    def _use(self, *names):
        """With offload enabled keep only the named models on the GPU (pipelines/base.py:96-122)."""
        if not self.cpu_offload:
            return
        for n in ("text_encoder", "image_encoder", "dit", "vae"):
            m = getattr(self, n)
            if m is not None:
                m.to(self.device if n in names else "cpu")
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    # ---- stages -----------------------------------------------------------------------------------
    def check_resize_height_width(self, height, width):
        h = height // self.height_division_factor * self.height_division_factor
        w = width // self.width_division_factor * self.width_division_factor
        return h, w

    def encode_prompt(self, prompt: str, text_len: int = 512):
        ids, mask = self.tokenizer([prompt])
        ids, mask = ids[:, :text_len].to(self.device), mask[:, :text_len].to(self.device)
        return {"context": encode_prompt(self.text_encoder, ids, mask).to(self.torch_dtype)}

    def preprocess_image(self, image) -> torch.Tensor:
        """PIL image or [3,H,W] / [H,W,3] array in 0..255 or [-1,1] -> [1,3,H,W] in [-1,1]."""
        if torch.is_tensor(image):
            t = image.float()
        else:
            import numpy as np

            t = torch.from_numpy(np.asarray(image)).float()
        if t.dim() == 3 and t.shape[-1] == 3:
            t = t.permute(2, 0, 1)
        if t.max() > 1.5:
            t = t / 127.5 - 1.0
        return t.unsqueeze(0)

    def encode_image(self, image, num_frames, height, width, end_image=None):
        img = torch.nn.functional.interpolate(self.preprocess_image(image), size=(height, width), mode="bilinear")
        img = img.to(self.device, self.torch_dtype)
        clip = self.image_encoder.encode_image(img)
        f, h, w = (num_frames - 1) // 4 + 1, height // 8, width // 8
        msk = torch.zeros(1, 4, f, h, w, device=self.device, dtype=self.torch_dtype)
        msk[:, :, 0] = 1
        vid = torch.cat([img.unsqueeze(2), torch.zeros(1, 3, num_frames - 1, height, width, device=self.device,
                                                       dtype=self.torch_dtype)], dim=2)
        if end_image is not None:
            end = torch.nn.functional.interpolate(self.preprocess_image(end_image), size=(height, width),
                                                  mode="bilinear").to(self.device, self.torch_dtype)
            vid[:, :, -1] = end[:, :]
            msk[:, :, -1] = 1
            clip = torch.cat([clip, self.image_encoder.encode_image(end)], dim=1)
        y = self.vae.encode(list(vid), device=self.device)
        return {"clip_feature": clip.to(self.torch_dtype), "y": torch.cat([msk, y.to(self.torch_dtype)], dim=1)}

    def tensor2video(self, frames: torch.Tensor) -> List:
        """[3, T, H, W] in [-1,1] -> list of PIL images (numpy arrays when PIL is missing)."""
        arr = ((frames.float().clamp(-1, 1) + 1) * 127.5).round().byte().permute(1, 2, 3, 0).cpu().numpy()
        try:
            from PIL import Image

            return [Image.fromarray(a) for a in arr]
        except Exception:
            return list(arr)

    # ---- sampling ---------------------------------------------------------------------------------
    @torch.no_grad()
    def __call__(self, prompt, negative_prompt="", input_image=None, end_image=None, input_video=None,
                 denoising_strength=1.0, seed=None, rand_device="cpu", height=480, width=832, num_frames=81,
                 cfg_scale=5.0, num_inference_steps=50, sigma_shift=5.0, tiled=True, tile_size=(30, 52),
                 tile_stride=(15, 26), progress_bar_cmd=lambda x: x, output_type="pil", tea_cache_l1_thresh=None,
                 tea_cache_coefficients=None):
        height, width = self.check_resize_height_width(height, width)
        if num_frames % 4 != 1:
            num_frames = (num_frames + 2) // 4 * 4 + 1
        self.scheduler.set_timesteps(num_inference_steps, denoising_strength=denoising_strength, shift=sigma_shift)
        gen = None if seed is None else torch.Generator(device=rand_device).manual_seed(seed)
        shape = (1, 16, (num_frames - 1) // 4 + 1, height // 8, width // 8)
        noise = torch.randn(shape, generator=gen, device=rand_device, dtype=torch.float32).to(self.device, self.torch_dtype)
        if input_video is not None:                       # video-to-video: start from a noised encoding
            self._use("vae")
            vid = torch.stack([self.preprocess_image(f)[0] for f in input_video], dim=1).to(self.device, self.torch_dtype)
            lat = self.vae.encode([vid], device=self.device, tiled=tiled, tile_size=tile_size,
                                  tile_stride=tile_stride).to(self.torch_dtype)
            latents = self.scheduler.add_noise(lat, noise, self.scheduler.timesteps[0])
        else:
            latents = noise
        self._use("text_encoder")
        pos = self.encode_prompt(prompt)
        neg = self.encode_prompt(negative_prompt) if cfg_scale != 1.0 else None
        extra = {}
        if input_image is not None and self.image_encoder is not None:
            self._use("image_encoder", "vae")
            extra = self.encode_image(input_image, num_frames, height, width, end_image)
        self._use("dit")
        self.dit.eval()
        caches = None
        if tea_cache_l1_thresh is not None:
            n_steps = len(self.scheduler.timesteps)
            caches = [StepCache(n_steps, tea_cache_l1_thresh, tea_cache_coefficients) for _ in range(2)]
        self.last_step_caches = caches

        def run(branch, ts, ctx):
            if caches is not None:
                from ..models.wan import sinusoidal_embedding_1d

                emb = self.dit._small_mlp(self.dit.time_embedding,
                                          sinusoidal_embedding_1d(self.dit.cfg.freq_dim, ts.to(self.device)))
                if caches[branch].should_skip(self.dit._small_mlp(self.dit.time_projection, emb)):
                    return caches[branch].last_out
            out = self.dit(latents, ts, ctx, extra.get("clip_feature"), extra.get("y"))
            if caches is not None:
                caches[branch].last_out = out
            return out

        for t in progress_bar_cmd(self.scheduler.timesteps):
            ts = t.reshape(1).to(self.device, torch.float32)
            v_pos = run(0, ts, pos["context"])
            if neg is not None:
                v_neg = run(1, ts, neg["context"])
                v = v_neg + cfg_scale * (v_pos - v_neg)
            else:
                v = v_pos
            latents = self.scheduler.step(v.float(), t, latents.float()).to(self.torch_dtype)
        self._use("vae")
        frames = self.vae.decode(latents, device=self.device, tiled=tiled, tile_size=tile_size, tile_stride=tile_stride)
        self._use()
        if output_type == "latent":
            return latents
        if output_type == "tensor":
            return frames[0]
        return self.tensor2video(frames[0])
