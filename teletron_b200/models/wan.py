"""Wan2.1 video DiT (t2v / i2v, 1.3B / 14B from config) on the teletron_b200 op layer.

Architecture and state-dict key names follow the reference DiT
(teletron/models/wan/wan_model.py:137-396): patch embedding (a (1,2,2) Conv3d = reshape +
GEMM), text / time embedders, N blocks of [AdaLN -> self-attention with full-width q/k
RMSNorm and 3-axis RoPE -> gated residual; affine LN -> cross-attention (text, plus CLIP
image tokens for i2v) -> residual; AdaLN -> GELU-tanh FFN -> gated residual] and a modulated
head.  Differences by design:
  * q/k/v (and cross-attention k/v) are one fused projection; the state dict still exposes
    ``q/k/v.weight`` so reference checkpoints load unchanged.
  * the hidden state is a 2-D ``[batch*tokens, C]`` bf16 matrix; modulation vectors stay fp32.
  * RoPE is a cached fp32 (cos, sin) table, built once per latent grid in float64.
  * under Ulysses context parallelism the sequence is split right after the patch
    embedding and the loss can be taken on the local shard, so every parameter gradient is a
    partial sum over the CP group (no per-parameter all-gather hooks as in
    teletron/models/wan/parallel_wan_model.py:62-74).
  * shapes come from ``WanConfig`` rather than a hard-coded class
    (teletron/models/wan/wan_model.py:29-41).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel import recompute as rc
from ..parallel.ulysses import UlyssesContext

T5_CONTEXT_TOKENS = 512


@dataclass
class WanConfig:
    dim: int = 1536
    num_heads: int = 12
    num_layers: int = 30
    ffn_dim: int = 8960
    in_dim: int = 16
    out_dim: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    eps: float = 1e-6
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    has_image_input: bool = False
    has_image_pos_emb: bool = False
    clip_dim: int = 1280
    rope_max_pos: int = 1024
    # activation recompute: None | "full"; method "uniform" | "block"; number of layers
    recompute_granularity: Optional[str] = None
    recompute_method: str = "block"
    recompute_num_layers: int = 0
    activation_offload: bool = False

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads


WAN_PRESETS = {
    "wan2.1-1.3b-t2v": dict(dim=1536, num_heads=12, num_layers=30, ffn_dim=8960, in_dim=16),
    "wan2.1-14b-t2v": dict(dim=5120, num_heads=40, num_layers=40, ffn_dim=13824, in_dim=16),
    "wan2.1-14b-i2v": dict(dim=5120, num_heads=40, num_layers=40, ffn_dim=13824, in_dim=36,
                           has_image_input=True),
    "wan-tiny": dict(dim=128, num_heads=4, num_layers=2, ffn_dim=512, in_dim=16, text_dim=64,
                     freq_dim=64),
}


def wan_config(name: str, **overrides) -> WanConfig:
    cfg = dict(WAN_PRESETS[name])
    cfg.update(overrides)
    return WanConfig(**cfg)


# ------------------------------------------------------------------------- embeddings
def sinusoidal_embedding_1d(dim: int, position: torch.Tensor) -> torch.Tensor:
    """[B] -> [B, dim] (cos | sin), computed in float64 like the reference (wan_model.py:81-85)."""
    pos = position.to(torch.float64)
    half = dim // 2
    freqs = torch.pow(10000.0, -torch.arange(half, dtype=torch.float64, device=pos.device) / half)
    ang = torch.outer(pos, freqs)
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).float()


def rope_table_3d(head_dim: int, grid: Tuple[int, int, int], theta: float = 10000.0,
                  device=None) -> torch.Tensor:
    """fp32 [f*h*w, head_dim/2, 2] of (cos, sin): frame axis gets d - 2*(d//3) dims, height and
    width d//3 each (wan_model.py:88-102), token order (f, h, w) row-major."""
    f, h, w = grid
    d_h = d_w = head_dim // 3
    d_f = head_dim - 2 * (head_dim // 3)

    def axis(dim, n):
        fr = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64)[: dim // 2] / dim))
        return torch.outer(torch.arange(n, dtype=torch.float64), fr)  # [n, dim/2]

    af, ah, aw = axis(d_f, f), axis(d_h, h), axis(d_w, w)
    ang = torch.cat([
        af.view(f, 1, 1, -1).expand(f, h, w, -1),
        ah.view(1, h, 1, -1).expand(f, h, w, -1),
        aw.view(1, 1, w, -1).expand(f, h, w, -1),
    ], dim=-1).reshape(f * h * w, -1)
    tab = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()
    return tab.to(device) if device is not None else tab


class FusedProj(nn.Module):
    """One [n*dim_out, dim_in] projection that appears in the state dict as n separate Linear
    layers (``names``), so fused q/k/v storage stays checkpoint-compatible."""

    def __init__(self, dim_in: int, dim_out: int, names: Tuple[str, ...]):
        super().__init__()
        self.names = names
        self.dim_out = dim_out
        self.weight = nn.Parameter(torch.empty(len(names) * dim_out, dim_in))
        self.bias = nn.Parameter(torch.zeros(len(names) * dim_out))
        for i in range(len(names)):
            nn.init.kaiming_uniform_(self.weight.data[i * dim_out:(i + 1) * dim_out], a=math.sqrt(5))
        bound = 1.0 / math.sqrt(dim_in)
        nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x2d):
        return ops.linear(x2d, self.weight, self.bias)


def _split_fused_state(module: nn.Module, state, prefix: str, fused_attr: str):
    """state-dict save hook helper: replace `<prefix><fused_attr>.weight` by per-name entries."""
    fp: FusedProj = getattr(module, fused_attr)
    for kind in ("weight", "bias"):
        key = f"{prefix}{fused_attr}.{kind}"
        if key in state:
            t = state.pop(key)
            for i, n in enumerate(fp.names):
                state[f"{prefix}{n}.{kind}"] = t[i * fp.dim_out:(i + 1) * fp.dim_out]


def _merge_fused_state(module: nn.Module, state, prefix: str, fused_attr: str):
    fp: FusedProj = getattr(module, fused_attr)
    for kind in ("weight", "bias"):
        keys = [f"{prefix}{n}.{kind}" for n in fp.names]
        if all(k in state for k in keys):
            state[f"{prefix}{fused_attr}.{kind}"] = torch.cat([state.pop(k) for k in keys], dim=0)


class _FusedStateMixin:
    _fused_attrs: Tuple[str, ...] = ()

    def _install_fused_hooks(self):
        def save_hook(module, state, prefix, _local):
            for a in module._fused_attrs:
                _split_fused_state(module, state, prefix, a)
            return state

        def load_hook(module, state, prefix, *_):
            for a in module._fused_attrs:
                _merge_fused_state(module, state, prefix, a)

        self._register_state_dict_hook(save_hook)
        self.register_load_state_dict_pre_hook(load_hook)


class RMSNormWeight(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))


class SelfAttention(nn.Module, _FusedStateMixin):
    _fused_attrs = ("qkv",)

    def __init__(self, dim: int, num_heads: int, eps: float):
        super().__init__()
        self.dim, self.num_heads, self.head_dim, self.eps = dim, num_heads, dim // num_heads, eps
        self.qkv = FusedProj(dim, dim, ("q", "k", "v"))
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNormWeight(dim)
        self.norm_k = RMSNormWeight(dim)
        self._install_fused_hooks()

    def forward(self, h2d, freqs, batch, cp: Optional[UlyssesContext], residual, gate, rows_per_batch):
        C, H, D = self.dim, self.num_heads, self.head_dim
        fu = cp.fused if (cp is not None and cp.size > 1) else None
        if fu is not None and h2d.is_cuda and fu.supports(H, D):
            # all-to-alls fused into the projection GEMM's, the norm/rope kernel's and the attention kernel's stores
            # (peer memory)
            fu.seq_len = cp.seq_len
            a2d = fu.attention_qkv(h2d, self.qkv.weight, self.qkv.bias, self.norm_q.weight, self.norm_k.weight,
                                   freqs, batch, rows_per_batch, H, D, self.eps)
            return ops.linear_residual(a2d, self.o.weight, self.o.bias, residual, gate, rows_per_batch)
        qkv = self.qkv(h2d)  # [rows, 3C]
        S = rows_per_batch
        if cp is None or cp.size == 1:
            # norm + rope + attention as one autograd node on the three column blocks of qkv
            a2d = ops.self_attention_core(qkv, self.norm_q.weight, self.norm_k.weight, freqs, batch, S, H, D, self.eps)
            return ops.linear_residual(a2d, self.o.weight, self.o.bias, residual, gate, rows_per_batch)
        q = ops.rmsnorm_rope(qkv[:, 0:C], self.norm_q.weight, freqs, D, False, self.eps)
        k = ops.rmsnorm_rope(qkv[:, C:2 * C], self.norm_k.weight, freqs, D, False, self.eps)
        v = qkv[:, 2 * C:3 * C]
        q4 = q.view(batch, S, H, D)
        k4 = k.view(batch, S, H, D)
        v4 = v.unflatten(1, (H, D)).unflatten(0, (batch, S))
        a = cp.attention(q4, k4, v4)
        a2d = a.reshape(batch * S, C)
        return ops.linear_residual(a2d, self.o.weight, self.o.bias, residual, gate, rows_per_batch)


class CrossAttention(nn.Module, _FusedStateMixin):
    def __init__(self, dim: int, num_heads: int, eps: float, has_image_input: bool):
        super().__init__()
        self.dim, self.num_heads, self.head_dim, self.eps = dim, num_heads, dim // num_heads, eps
        self.has_image_input = has_image_input
        self.q = nn.Linear(dim, dim)
        self.kv = FusedProj(dim, dim, ("k", "v"))
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNormWeight(dim)
        self.norm_k = RMSNormWeight(dim)
        self._fused_attrs = ("kv",)
        if has_image_input:
            self.kv_img = FusedProj(dim, dim, ("k_img", "v_img"))
            self.norm_k_img = RMSNormWeight(dim)
            self._fused_attrs = ("kv", "kv_img")
        self._install_fused_hooks()

    def forward(self, h2d, context, batch, residual, rows_per_batch):
        C, H, D = self.dim, self.num_heads, self.head_dim
        S = rows_per_batch
        if self.has_image_input:
            n_img = context.shape[1] - T5_CONTEXT_TOKENS
            img, ctx = context[:, :n_img], context[:, n_img:]
        else:
            img, ctx = None, context
        q = ops.rmsnorm_rope(ops.linear(h2d, self.q.weight, self.q.bias), self.norm_q.weight, None, D,
                             False, self.eps)
        q4 = q.view(batch, S, H, D)

        def kv_of(tokens, proj, norm):
            Lc = tokens.shape[1]
            kv = proj(tokens.reshape(batch * Lc, C))
            k = ops.rmsnorm_rope(kv[:, 0:C], norm.weight, None, D, False, self.eps)
            return k.view(batch, Lc, H, D), kv[:, C:2 * C].unflatten(1, (H, D)).unflatten(0, (batch, Lc))

        k4, v4 = kv_of(ctx, self.kv, self.norm_k)
        a = ops.attention(q4, k4, v4)
        if img is not None:
            ki, vi = kv_of(img, self.kv_img, self.norm_k_img)
            a = a + ops.attention(q4, ki, vi)
        return ops.linear_residual(a.reshape(batch * S, C), self.o.weight, self.o.bias, residual, None,
                                   rows_per_batch)


class DiTBlock(nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        dim = cfg.dim
        self.dim, self.eps = dim, cfg.eps
        self.self_attn = SelfAttention(dim, cfg.num_heads, cfg.eps)
        self.cross_attn = CrossAttention(dim, cfg.num_heads, cfg.eps, cfg.has_image_input)
        self.norm3 = nn.LayerNorm(dim, eps=cfg.eps)
        self.ffn = nn.Sequential(nn.Linear(dim, cfg.ffn_dim), nn.GELU(approximate="tanh"),
                                 nn.Linear(cfg.ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

    def forward(self, x2d, context, t_mod, freqs, batch: int, cp: Optional[UlyssesContext]):
        rows_per_batch = x2d.shape[0] // batch
        e = self.modulation.float() + t_mod  # [B, 6, C] fp32
        # each norm also hands back its input for the residual branch, so that the residual's gradient is added
        # inside the norm's backward kernel
        h, xr = ops.adaln_res(x2d, e[:, 1], e[:, 0], rows_per_batch, self.eps)
        x2d = self.self_attn(h, freqs, batch, cp, xr, e[:, 2], rows_per_batch)
        h, xr = ops.layernorm_affine(x2d, self.norm3.weight, self.norm3.bias, self.eps, with_res=True)
        x2d = self.cross_attn(h, context, batch, xr, rows_per_batch)
        h, xr = ops.adaln_res(x2d, e[:, 4], e[:, 3], rows_per_batch, self.eps)
        return ops.ffn(h, self.ffn[0].weight, self.ffn[0].bias, self.ffn[2].weight, self.ffn[2].bias, xr, e[:, 5],
                       rows_per_batch, act="gelu")


class ImageEmbedMLP(nn.Module):
    """CLIP-token embedder of the i2v model (wan_model.py:246-263); small, plain PyTorch."""

    def __init__(self, in_dim, out_dim, has_pos_emb=False):
        super().__init__()
        self.proj = nn.Sequential(nn.LayerNorm(in_dim), nn.Linear(in_dim, in_dim), nn.GELU(),
                                  nn.Linear(in_dim, out_dim), nn.LayerNorm(out_dim))
        self.has_pos_emb = has_pos_emb
        if has_pos_emb:
            self.emb_pos = nn.Parameter(torch.zeros((1, 514, 1280)))

    def forward(self, x):
        if self.has_pos_emb:
            x = x + self.emb_pos.to(dtype=x.dtype, device=x.device)
        return self.proj(x)


class Head(nn.Module):
    def __init__(self, dim, out_dim, patch_size, eps):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.head = nn.Linear(dim, out_dim * math.prod(patch_size))
        self.modulation = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)

    def forward(self, x2d, t, batch):
        rows_per_batch = x2d.shape[0] // batch
        e = self.modulation.float() + t.float().unsqueeze(1)  # [B, 2, C]
        h = ops.adaln(x2d, e[:, 1], e[:, 0], rows_per_batch, self.eps)
        return ops.linear(h, self.head.weight, self.head.bias)


class WanModel(nn.Module):
    """forward(x, timestep, context, clip_feature=None, y=None) -> velocity prediction with the
    same signature as ParallelWanModel.forward (teletron/models/wan/parallel_wan_model.py:76-117)."""

    def __init__(self, cfg: WanConfig, cp: Optional[UlyssesContext] = None):
        super().__init__()
        self.cfg = cfg
        self.cp = cp
        dim = cfg.dim
        self.patch_embedding = nn.Conv3d(cfg.in_dim, dim, kernel_size=cfg.patch_size, stride=cfg.patch_size)
        self.text_embedding = nn.Sequential(nn.Linear(cfg.text_dim, dim), nn.GELU(approximate="tanh"),
                                            nn.Linear(dim, dim))
        self.time_embedding = nn.Sequential(nn.Linear(cfg.freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(dim, dim * 6))
        self.blocks = nn.ModuleList([DiTBlock(cfg) for _ in range(cfg.num_layers)])
        self.head = Head(dim, cfg.out_dim, cfg.patch_size, cfg.eps)
        if cfg.has_image_input:
            self.img_emb = ImageEmbedMLP(cfg.clip_dim, dim, cfg.has_image_pos_emb)
        self._rope_cache = {}
        self.return_local_shard = False  # CP: skip the output gather (loss on the local tokens)

    # --- token <-> latent layout -------------------------------------------------------
    def patchify(self, x):
        """[B, Cin, F, H, W] -> ([B*S, Cin*pt*ph*pw], (f, h, w)) in conv-weight element order."""
        B, Cin, Fr, Hh, Ww = x.shape
        pt, ph, pw = self.cfg.patch_size
        f, h, w = Fr // pt, Hh // ph, Ww // pw
        p = x.reshape(B, Cin, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return p.reshape(B * f * h * w, Cin * pt * ph * pw), (f, h, w)

    def unpatchify(self, x, grid):
        """[B, S, pt*ph*pw*Cout] -> [B, Cout, F, H, W] ('(x y z c)' ordering of the head output)."""
        f, h, w = grid
        pt, ph, pw = self.cfg.patch_size
        B = x.shape[0]
        x = x.reshape(B, f, h, w, pt, ph, pw, self.cfg.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(B, self.cfg.out_dim, f * pt, h * ph, w * pw)

    def rope(self, grid, device):
        key = (tuple(grid), str(device))
        tab = self._rope_cache.get(key)
        if tab is None:
            tab = rope_table_3d(self.cfg.head_dim, grid, device=device)
            self._rope_cache[key] = tab
        return tab

    def _small_mlp(self, seq: nn.Sequential, x):
        """Tiny per-sample MLPs (time embedding / projection) in fp32."""
        for m in seq:
            if isinstance(m, nn.Linear):
                x = F.linear(x, m.weight.float(), m.bias.float())
            else:
                x = m(x)
        return x

    def forward(self, x, timestep, context, clip_feature=None, y=None, **_unused):
        cfg = self.cfg
        dt = self.patch_embedding.weight.dtype
        B = x.shape[0]
        t = self._small_mlp(self.time_embedding, sinusoidal_embedding_1d(cfg.freq_dim, timestep.to(x.device)))
        t_mod = self._small_mlp(self.time_projection, t).unflatten(1, (6, cfg.dim))  # fp32 [B,6,C]
        Lc = context.shape[1]
        ctx = context.to(dt).reshape(B * Lc, cfg.text_dim)
        ctx = ops.linear(ctx, self.text_embedding[0].weight, self.text_embedding[0].bias, act="gelu")
        ctx = ops.linear(ctx, self.text_embedding[2].weight, self.text_embedding[2].bias).view(B, Lc, cfg.dim)
        if cfg.has_image_input:
            x = torch.cat([x, y.to(x.dtype)], dim=1)
            ctx = torch.cat([self.img_emb(clip_feature.to(dt)), ctx], dim=1)
        patches, grid = self.patchify(x.to(dt))
        S = grid[0] * grid[1] * grid[2]
        w2d = self.patch_embedding.weight.view(cfg.dim, -1)
        tok = ops.linear(patches.contiguous(), w2d, self.patch_embedding.bias)  # [B*S, C]
        freqs = self.rope(grid, x.device)
        cp = self.cp if (self.cp is not None and self.cp.size > 1) else None
        if cp is not None:
            tok = cp.split_tokens(tok.view(B, S, cfg.dim)).reshape(-1, cfg.dim)
            freqs = cp.split_rows(freqs)
            fu = cp.fused
            if fu is not None and tok.is_cuda and fu.supports(cfg.num_heads, cfg.head_dim):
                alive = cfg.num_layers
                if self.training and cfg.recompute_granularity == "full":
                    k = cfg.recompute_num_layers or 1
                    alive = (cfg.num_layers - min(k, cfg.num_layers) + 2) if cfg.recompute_method == "block" else k + 1
                fu.begin_microbatch(fu.slab_elems(alive, B, cp.padded_len(S), cfg.dim, cp.size))
        tok = rc.run_blocks(self.blocks, tok, (ctx, t_mod, freqs, B, cp), cfg, self.training)
        out = self.head(tok, t, B)  # [B*S_local, 64]
        out = out.view(B, -1, out.shape[-1])
        if cp is not None:
            if self.return_local_shard:
                return out
            out = cp.gather_tokens(out, S)
        return self.unpatchify(out, grid)

    def local_target_tokens(self, latents):
        """Lay a latent-shaped tensor out as this rank's [B, S_local, pt*ph*pw*Cout] token shard, the
        layout `forward` returns when ``return_local_shard`` is set."""
        B, Cc, Fr, Hh, Ww = latents.shape
        pt, ph, pw = self.cfg.patch_size
        f, h, w = Fr // pt, Hh // ph, Ww // pw
        tk = latents.reshape(B, Cc, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 3, 5, 7, 1)
        tk = tk.reshape(B, f * h * w, pt * ph * pw * Cc)
        if self.cp is not None and self.cp.size > 1:
            tk = self.cp.split_tokens(tk)
        return tk
