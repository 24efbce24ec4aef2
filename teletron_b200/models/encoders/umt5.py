"""umT5-XXL-shaped text encoder (encoder stack only): 24 layers, d_model 4096, 64 heads of 64,
gated-GELU FFN 10240, T5 layer norm (RMS, no bias), per-layer relative position bias with 32
bidirectional buckets, vocabulary 256384.

Module names follow the reference text encoder (teletron/models/wan/encoder/
wan_video_text_encoder.py:210-255): ``token_embedding``, ``blocks.N.{norm1, attn.{q,k,v,o}, pos_embedding.
embedding, norm2, ffn.{gate.0, fc1, fc2}}``, ``norm``.  Plain PyTorch: the encoder runs once per
sample on dedicated encoder ranks, not on the DiT hot path.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class T5LayerNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf.to(x.dtype)) * self.weight


class T5RelativeEmbedding(nn.Module):
    def __init__(self, num_buckets, num_heads, bidirectional=True, max_dist=128):
        super().__init__()
        self.num_buckets, self.num_heads, self.bidirectional, self.max_dist = num_buckets, num_heads, bidirectional, max_dist
        self.embedding = nn.Embedding(num_buckets, num_heads)

    def _bucket(self, rel):
        if self.bidirectional:
            nb = self.num_buckets // 2
            out = (rel > 0).long() * nb
            rel = rel.abs()
        else:
            nb = self.num_buckets
            out = torch.zeros_like(rel)
            rel = -torch.min(rel, torch.zeros_like(rel))
        max_exact = nb // 2
        large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(self.max_dist / max_exact)
                             * (nb - max_exact)).long()
        large = torch.min(large, torch.full_like(large, nb - 1))
        return out + torch.where(rel < max_exact, rel, large)

    def forward(self, lq, lk):
        dev = self.embedding.weight.device
        rel = torch.arange(lk, device=dev).unsqueeze(0) - torch.arange(lq, device=dev).unsqueeze(1)
        return self.embedding(self._bucket(rel)).permute(2, 0, 1).unsqueeze(0)  # [1, heads, lq, lk]


class T5Attention(nn.Module):
    def __init__(self, dim, dim_attn, num_heads):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, dim_attn // num_heads
        self.q = nn.Linear(dim, dim_attn, bias=False)
        self.k = nn.Linear(dim, dim_attn, bias=False)
        self.v = nn.Linear(dim, dim_attn, bias=False)
        self.o = nn.Linear(dim_attn, dim, bias=False)

    def forward(self, x, mask=None, pos_bias=None):
        b, n, c = x.shape[0], self.num_heads, self.head_dim
        q = self.q(x).view(b, -1, n, c).transpose(1, 2)
        k = self.k(x).view(b, -1, n, c).transpose(1, 2)
        v = self.v(x).view(b, -1, n, c).transpose(1, 2)
        bias = torch.zeros(b, n, q.shape[2], k.shape[2], dtype=q.dtype, device=q.device)
        if pos_bias is not None:
            bias = bias + pos_bias.to(q.dtype)
        if mask is not None:
            m = mask.view(b, 1, 1, -1) if mask.dim() == 2 else mask.unsqueeze(1)
            bias = bias.masked_fill(m == 0, torch.finfo(q.dtype).min)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, scale=1.0)  # T5 does not scale by 1/sqrt(d)
        return self.o(o.transpose(1, 2).reshape(b, -1, n * c))


class T5FeedForward(nn.Module):
    def __init__(self, dim, dim_ffn):
        super().__init__()
        self.gate = nn.Sequential(nn.Linear(dim, dim_ffn, bias=False), nn.GELU(approximate="tanh"))
        self.fc1 = nn.Linear(dim, dim_ffn, bias=False)
        self.fc2 = nn.Linear(dim_ffn, dim, bias=False)

    def forward(self, x):
        return self.fc2(self.fc1(x) * self.gate(x))


class T5SelfAttentionBlock(nn.Module):
    def __init__(self, dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos):
        super().__init__()
        self.norm1 = T5LayerNorm(dim)
        self.attn = T5Attention(dim, dim_attn, num_heads)
        self.norm2 = T5LayerNorm(dim)
        self.ffn = T5FeedForward(dim, dim_ffn)
        self.pos_embedding = None if shared_pos else T5RelativeEmbedding(num_buckets, num_heads, True)

    def forward(self, x, mask=None, pos_bias=None):
        e = pos_bias if self.pos_embedding is None else self.pos_embedding(x.shape[1], x.shape[1])
        x = x + self.attn(self.norm1(x), mask=mask, pos_bias=e)
        return x + self.ffn(self.norm2(x))


class UMT5Encoder(nn.Module):
    def __init__(self, vocab=256384, dim=4096, dim_attn=4096, dim_ffn=10240, num_heads=64, num_layers=24,
                 num_buckets=32, shared_pos=False):
        super().__init__()
        self.dim = dim
        self.token_embedding = nn.Embedding(vocab, dim)
        self.pos_embedding = T5RelativeEmbedding(num_buckets, num_heads, True) if shared_pos else None
        self.blocks = nn.ModuleList([T5SelfAttentionBlock(dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos)
                                     for _ in range(num_layers)])
        self.norm = T5LayerNorm(dim)

    def forward(self, ids, mask=None):
        x = self.token_embedding(ids)
        e = self.pos_embedding(x.shape[1], x.shape[1]) if self.pos_embedding is not None else None
        for blk in self.blocks:
            x = blk(x, mask, pos_bias=e)
        return self.norm(x)


def encode_prompt(encoder: UMT5Encoder, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """[B, L] ids/mask -> [B, L, dim] with positions past each prompt's length zeroed
    (teletron/models/wan/encoder/wan_prompter.py:101-111)."""
    out = encoder(ids, mask)
    lens = mask.gt(0).sum(dim=1)
    keep = torch.arange(ids.shape[1], device=ids.device)[None, :] < lens[:, None]
    return out * keep.unsqueeze(-1).to(out.dtype)
