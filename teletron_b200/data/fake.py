"""Synthetic datasets.

``FakeDataset`` yields what the reference's does (teletron/datasets/fake_dataset.py:8-41): a random
prompt string, a random video ``images [T,3,H,W]`` and its first frame — the raw inputs of the
encoder ranks.  ``SyntheticLatentDataset`` yields already-encoded samples (latents, umT5-shaped
context, optional CLIP tokens and image-condition latent) with the shapes of a given
resolution, which is what benchmarks and encoder-less training use.  Items are generated
from the index, so every rank/worker sees the same sample for the same index.
"""
from __future__ import annotations

import string

import torch
from torch.utils.data import Dataset

from .registry import DATASETS


def latent_grid(num_frames: int, height: int, width: int):
    """(frames, h, w) of the VAE latent: 4x temporal (1 + (F-1)/4), 8x spatial compression."""
    return (num_frames - 1) // 4 + 1, height // 8, width // 8


@DATASETS.register("FakeDataset")
class FakeDataset(Dataset):
    def __init__(self, num_frames=81, height=480, width=832, length=10_000_000, prompt_len=880, seed=0, **_):
        self.num_frames, self.height, self.width = num_frames, height, width
        self.length, self.prompt_len, self.seed = length, prompt_len, seed

    def __len__(self):
        return self.length

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + int(idx))
        letters = string.ascii_lowercase + " "
        ids = torch.randint(0, len(letters), (self.prompt_len,), generator=g)
        prompt = "".join(letters[i] for i in ids.tolist())
        images = torch.randn(self.num_frames, 3, self.height, self.width, generator=g)
        return dict(prompts=prompt, images=images, raw_first_image=images[0].clone(), index=int(idx))


@DATASETS.register("SyntheticLatentDataset")
class SyntheticLatentDataset(Dataset):
    def __init__(self, num_frames=81, height=480, width=832, length=10_000_000, text_len=512, text_dim=4096,
                 i2v=False, clip_tokens=257, clip_dim=1280, dtype=torch.bfloat16, seed=0, fixed_noise=False,
                 train_timesteps=1000, **_):
        """``fixed_noise``: every item also carries its own ``noise`` and ``timestep_id`` (functions of the index),
        so that the loss of a global batch does not depend on how the batch is split over ranks and micro-batches
        (parity checks across parallel layouts)."""
        self.grid = latent_grid(num_frames, height, width)
        self.length, self.text_len, self.text_dim = length, text_len, text_dim
        self.i2v, self.clip_tokens, self.clip_dim, self.dtype, self.seed = i2v, clip_tokens, clip_dim, dtype, seed
        self.fixed_noise, self.train_timesteps = fixed_noise, train_timesteps

    def __len__(self):
        return self.length

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + int(idx))
        f, h, w = self.grid
        out = dict(latents=torch.randn(16, f, h, w, generator=g).to(self.dtype),
                   context=torch.randn(self.text_len, self.text_dim, generator=g).to(self.dtype))
        if self.i2v:
            mask = torch.zeros(4, f, h, w)
            mask[:, 0] = 1.0
            cond = torch.randn(16, f, h, w, generator=g)
            out["image_emb_y"] = torch.cat([mask, cond], dim=0).to(self.dtype)
            out["clip_feature"] = torch.randn(self.clip_tokens, self.clip_dim, generator=g).to(self.dtype)
        if self.fixed_noise:
            out["noise"] = torch.randn(16, f, h, w, generator=g).to(self.dtype)
            out["timestep_id"] = torch.randint(0, self.train_timesteps, (), generator=g)
        return out


@DATASETS.register("SyntheticHunyuanDataset")
class SyntheticHunyuanDataset(Dataset):
    """Already-encoded HunyuanVideo samples in the order the encoder ranks deliver them (prompt_embeds,
    clip_text_embed, first_ref_image, latents): LLM text states ``[text_len, text_dim]`` with a ragged
    ``prompt_mask`` (the model masks the padded tail), the pooled CLIP text vector, the VAE latent of the first
    frame (image-to-video only) and the video latent."""

    def __init__(self, num_frames=129, height=720, width=1280, length=10_000_000, text_len=256, text_dim=4096,
                 pooled_dim=768, i2v=False, dtype=torch.bfloat16, seed=0, **_):
        self.grid = latent_grid(num_frames, height, width)
        self.length, self.text_len, self.text_dim, self.pooled_dim = length, text_len, text_dim, pooled_dim
        self.i2v, self.dtype, self.seed = i2v, dtype, seed

    def __len__(self):
        return self.length

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + int(idx))
        f, h, w = self.grid
        n_text = int(torch.randint(max(self.text_len // 4, 1), self.text_len + 1, (1,), generator=g))
        mask = torch.zeros(self.text_len, dtype=torch.long)
        mask[:n_text] = 1
        out = dict(latents=torch.randn(16, f, h, w, generator=g).to(self.dtype),
                   prompt_embeds=torch.randn(self.text_len, self.text_dim, generator=g).to(self.dtype),
                   prompt_mask=mask,
                   clip_text_embed=torch.randn(self.pooled_dim, generator=g).to(self.dtype))
        if self.i2v:
            out["first_ref_image"] = torch.randn(16, 1, h, w, generator=g).to(self.dtype)
        return out
