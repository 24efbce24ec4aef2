"""CLIP ViT-H/14 image encoder as used for Wan i2v conditioning: 224x224 input, 16x16 patches + class
token (257 tokens), width 1280, 32 pre-LN transformer blocks of 16 heads with a 5120-wide GELU MLP;
the conditioning features are the tokens after the second-to-last block
(teletron/models/wan/encoder/wan_video_image_encoder.py:388-480,824-882).  Plain PyTorch (runs on
encoder ranks).  Parameter names: ``visual.{patch_embedding, cls_embedding, pos_embedding, pre_norm,
transformer.N.{norm1, attn.{to_qkv, proj}, norm2, mlp.{0,2}}, post_norm}``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class ViTAttention(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads = heads
        self.to_qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        b, s, c = x.shape
        q, k, v = self.to_qkv(x).view(b, s, 3, self.heads, c // self.heads).permute(2, 0, 3, 1, 4)
        return self.proj(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, c))


class ViTBlock(nn.Module):
    def __init__(self, dim, heads, mlp_ratio=4, eps=1e-5):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=eps)
        self.attn = ViTAttention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, eps=eps)
        self.mlp = nn.Sequential(nn.Linear(dim, dim * mlp_ratio), nn.GELU(), nn.Linear(dim * mlp_ratio, dim))

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class VisionTransformer(nn.Module):
    def __init__(self, image_size=224, patch=14, dim=1280, heads=16, layers=32, mlp_ratio=4, out_dim=1024):
        super().__init__()
        self.image_size, self.patch = image_size, patch
        n = (image_size // patch) ** 2
        self.patch_embedding = nn.Conv2d(3, dim, patch, stride=patch, bias=False)
        self.cls_embedding = nn.Parameter(torch.randn(1, 1, dim) * dim ** -0.5)
        self.pos_embedding = nn.Parameter(torch.randn(1, n + 1, dim) * dim ** -0.5)
        self.pre_norm = nn.LayerNorm(dim, eps=1e-5)
        self.transformer = nn.Sequential(*[ViTBlock(dim, heads, mlp_ratio) for _ in range(layers)])
        self.post_norm = nn.LayerNorm(dim, eps=1e-5)
        self.head = nn.Parameter(torch.randn(dim, out_dim) * dim ** -0.5)

    def forward(self, x, use_31_block=True):
        b = x.shape[0]
        x = self.patch_embedding(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_embedding.expand(b, -1, -1).to(x.dtype), x], dim=1) + self.pos_embedding.to(x.dtype)
        x = self.pre_norm(x)
        if use_31_block:
            return self.transformer[:-1](x)          # penultimate-block tokens [B, 257, dim]
        return self.post_norm(self.transformer(x))


class WanImageEncoder(nn.Module):
    def __init__(self, dim=1280, layers=32, heads=16):
        super().__init__()
        self.model = nn.Module()
        self.model.visual = VisionTransformer(dim=dim, layers=layers, heads=heads)
        self.register_buffer("mean", torch.tensor(CLIP_MEAN).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("std", torch.tensor(CLIP_STD).view(1, 3, 1, 1), persistent=False)

    def reset_constants(self, device=None):
        """(Re)create the pixel normalisation constants (not part of any checkpoint)."""
        dev = device if device is not None else self.model.visual.patch_embedding.weight.device
        self.mean = torch.tensor(CLIP_MEAN, device=dev).view(1, 3, 1, 1)
        self.std = torch.tensor(CLIP_STD, device=dev).view(1, 3, 1, 1)

    @torch.no_grad()
    def encode_image(self, frames):
        """frames: [B, 3, H, W] in [-1, 1] -> CLIP tokens [B, 257, dim]."""
        size = self.model.visual.image_size
        x = F.interpolate(frames.float(), size=(size, size), mode="bicubic", align_corners=False)
        x = ((x * 0.5 + 0.5) - self.mean.to(x)) / self.std.to(x)
        return self.model.visual(x.to(self.model.visual.patch_embedding.weight.dtype), use_31_block=True)
