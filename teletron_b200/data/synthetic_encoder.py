"""A weight-free encoder for plumbing tests and benchmarks of the encoder service: it maps a raw
``FakeDataset`` item to tensors with the shapes and order of the Wan encoder output (context,
clip_feature, image_emb_y, latents[, noise]) using cheap deterministic projections instead of
umT5 / CLIP / VAE forward passes."""
from __future__ import annotations

import torch

from ..models.registry import ENCODERS
from .base_encoder import BaseEncoder
from .fake import latent_grid


@ENCODERS.register("synthetic_wan_encoder")
class SyntheticWanEncoder(BaseEncoder):
    def __init__(self, device=None, args=None, text_len=512, text_dim=4096, i2v=None, with_noise=None, **kw):
        super().__init__(device, **kw)
        self.text_len = getattr(args, "text_len", None) or text_len
        self.text_dim = getattr(args, "text_dim", None) or text_dim
        self.i2v = (getattr(args, "task_type", None) == "i2v") if i2v is None else i2v
        self.with_noise = (getattr(args, "consumer_models_num", 1) > 1) if with_noise is None else with_noise
        self.seq = 0

    def setup(self):
        return None

    def get_output_schema(self):
        return ["context", "clip_feature", "image_emb_y", "latents"] + (["noise"] if self.with_noise else [])

    def encode(self, raw_batch):
        images = raw_batch["images"]
        if images.dim() == 4:
            images = images.unsqueeze(0)
        B, T, _, H, W = images.shape
        f, h, w = latent_grid(T, H, W)
        idx = int(raw_batch["index"]) if not torch.is_tensor(raw_batch["index"]) else int(raw_batch["index"].reshape(-1)[0])
        g = torch.Generator().manual_seed(1_000_003 + idx)
        pooled = torch.nn.functional.adaptive_avg_pool3d(images.permute(0, 2, 1, 3, 4).float(), (f, h, w))
        latents = pooled.repeat(1, 6, 1, 1, 1)[:, :16] + 0.1 * torch.randn(B, 16, f, h, w, generator=g)
        context = torch.randn(B, self.text_len, self.text_dim, generator=g)
        if self.i2v:
            clip = torch.randn(B, 257, 1280, generator=g)
            mask = torch.zeros(B, 4, f, h, w)
            mask[:, :, 0] = 1.0
            y = torch.cat([mask, latents * mask[:, :1]], dim=1)
        else:
            clip = torch.zeros(B, 0, 1280)
            y = torch.zeros(B, 0, f, h, w)
        tensors = [context, clip, y, latents]
        if self.with_noise:
            tensors.append(torch.randn(B, 16, f, h, w, generator=g))
        tensors = [t.to(torch.bfloat16) for t in tensors]
        hdr = self._get_tensors_size(tensors, self.seq)
        self.seq += 1
        return tensors, hdr


@ENCODERS.register("synthetic_hunyuan_encoder")
class SyntheticHunyuanEncoder(BaseEncoder):
    """The HunyuanVideo counterpart: ``prompt_embeds [B, L, text_dim]``, ``clip_text_embed [B, pooled_dim]``,
    ``first_ref_image`` (first-frame latent ``[B, 16, 1, h, w]`` for image-to-video, empty otherwise) and
    ``latents``.  The reference ships no HunyuanVideo encoder bundle (LLM text encoder, CLIP-L, 3-D VAE); a real
    one is a ``BaseEncoder`` subclass with this output order, selected with ``--encoder-name``."""

    def __init__(self, device=None, args=None, text_len=256, text_dim=4096, pooled_dim=768, i2v=None, **kw):
        super().__init__(device, **kw)
        self.text_len = getattr(args, "text_len", None) or text_len
        self.text_dim = getattr(args, "text_embed_dim", None) or text_dim
        self.pooled_dim = getattr(args, "pooled_projection_dim", None) or pooled_dim
        preset = str(getattr(args, "model_preset", "") or "")
        if getattr(args, "text_embed_dim", None) is None and preset:
            from ..models.hunyuan import HUNYUAN_PRESETS

            self.text_dim = HUNYUAN_PRESETS.get(preset, {}).get("text_embed_dim", self.text_dim)
            self.pooled_dim = HUNYUAN_PRESETS.get(preset, {}).get("pooled_projection_dim", self.pooled_dim)
        self.i2v = (getattr(args, "task_type", None) == "i2v") if i2v is None else i2v
        self.seq = 0

    def setup(self):
        return None

    def get_output_schema(self):
        return ["prompt_embeds", "clip_text_embed", "first_ref_image", "latents"]

    def encode(self, raw_batch):
        images = raw_batch["images"]
        if images.dim() == 4:
            images = images.unsqueeze(0)
        B, T, _, H, W = images.shape
        f, h, w = latent_grid(T, H, W)
        idx = int(raw_batch["index"]) if not torch.is_tensor(raw_batch["index"]) else int(raw_batch["index"].reshape(-1)[0])
        g = torch.Generator().manual_seed(2_000_003 + idx)
        pooled = torch.nn.functional.adaptive_avg_pool3d(images.permute(0, 2, 1, 3, 4).float(), (f, h, w))
        latents = pooled.repeat(1, 6, 1, 1, 1)[:, :16] + 0.1 * torch.randn(B, 16, f, h, w, generator=g)
        text = torch.randn(B, self.text_len, self.text_dim, generator=g)
        clip = torch.randn(B, self.pooled_dim, generator=g)
        first = latents[:, :, :1].clone() if self.i2v else torch.zeros(B, 0, 1, h, w)
        tensors = [t.to(torch.bfloat16) for t in (text, clip, first, latents)]
        hdr = self._get_tensors_size(tensors, self.seq)
        self.seq += 1
        return tensors, hdr
