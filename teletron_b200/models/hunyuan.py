"""HunyuanVideo DiT (dual-stream + single-stream blocks) on the teletron_b200 op layer, with
Ulysses context parallelism and tensor parallelism built in.

The architecture and the state-dict key names follow the reference model, which is derived from
diffusers (teletron/models/hunyuan/model.py:45-995, parallel_model.py:35-390): timestep + guidance
+ pooled-text conditioning, a 2-layer token refiner for the text stream, N dual-stream blocks
(video and text have their own AdaLN / QKV / MLP and attend jointly), M single-stream blocks
(fused attention + MLP branch through one ``proj_out``), per-head q/k RMSNorm, RoPE (real cos/sin
on interleaved pairs, axes 16/56/56, theta 256) on video tokens only, and a key-length mask
for padded text.  It is written from scratch on this repo's ops, without diffusers.

Parallel design (differs from the reference, results are the same):
  * video tokens are sharded over the CP group after patch embedding; the text stream is
    replicated.  In joint attention the video q/k/v go through the seq->head exchange and each
    rank takes its own head slice of the replicated text q/k/v; afterwards the text heads are
    all-gathered with a reduce-scatter(sum) backward, which gives exact gradients without the
    reference's /P and xP scaling conventions (parallel_model.py:92-94,118).
  * padded text keys are masked by a per-sample key length inside the attention kernel instead
    of a dense [B, N, N] boolean mask (model.py:318-342).
  * tensor parallelism (absent from the reference's layers) shards heads and MLP width; see
    ``parallel/tp.py``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel import recompute as rc
from ..parallel.tp import ColumnParallelLinear, FusedColumnParallel, RowParallelLinear, TPContext
from ..parallel.ulysses import UlyssesContext, _HeadToSeq, _SeqToHead
from .registry import MODELS


@dataclass
class HunyuanConfig:
    hidden_size: int = 3072
    in_channels: int = 16
    out_channels: int = 16
    num_attention_heads: int = 24
    attention_head_dim: int = 128
    num_layers: int = 20            # dual-stream blocks
    num_single_layers: int = 40
    num_refiner_layers: int = 2
    mlp_ratio: float = 4.0
    patch_size: int = 2
    patch_size_t: int = 1
    guidance_embeds: bool = True
    text_embed_dim: int = 4096
    pooled_projection_dim: int = 768
    rope_theta: float = 256.0
    rope_axes_dim: Tuple[int, int, int] = (16, 56, 56)
    eps: float = 1e-6
    recompute_granularity: Optional[str] = None
    recompute_method: str = "block"
    recompute_num_layers: int = 0
    activation_offload: bool = False


HUNYUAN_PRESETS = {
    "hunyuanvideo-13b-t2v": dict(in_channels=16),
    "hunyuanvideo-13b-i2v": dict(in_channels=33),
    "hunyuan-tiny": dict(hidden_size=256, num_attention_heads=2, num_layers=1, num_single_layers=2,
                         num_refiner_layers=1, text_embed_dim=64, pooled_projection_dim=32),
}


def hunyuan_config(name: str, **kw) -> HunyuanConfig:
    c = dict(HUNYUAN_PRESETS[name])
    c.update(kw)
    return HunyuanConfig(**c)


# ------------------------------------------------------------------------------ embeddings
def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal features in (cos, sin) order with frequencies exp(-ln(max_period) * i / half)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1)


class TimestepEmbedder(nn.Module):
    def __init__(self, in_dim, dim):
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, dim)
        self.linear_2 = nn.Linear(dim, dim)

    def forward(self, x):
        x = F.linear(x.float(), self.linear_1.weight.float(), self.linear_1.bias.float())
        return F.linear(F.silu(x), self.linear_2.weight.float(), self.linear_2.bias.float())


class CombinedEmbeddings(nn.Module):
    """timestep (+ guidance) embedding plus projected pooled text; fp32, tiny."""

    def __init__(self, dim, pooled_dim, guidance: bool):
        super().__init__()
        self.timestep_embedder = TimestepEmbedder(256, dim)
        if guidance:
            self.guidance_embedder = TimestepEmbedder(256, dim)
        self.text_embedder = TimestepEmbedder(pooled_dim, dim)
        self.guidance = guidance

    def forward(self, timestep, pooled, guidance=None):
        c = self.timestep_embedder(timestep_embedding(timestep))
        if self.guidance:
            g = guidance if guidance is not None else torch.zeros_like(timestep)
            c = c + self.guidance_embedder(timestep_embedding(g))
        return c + self.text_embedder(pooled)


def hunyuan_rope_table(axes_dim, grid, theta: float, device=None) -> torch.Tensor:
    """fp32 [f*h*w, D/2, 2] (cos, sin) for token order (f, h, w); axis i uses axes_dim[i] dims."""
    f, h, w = grid
    sizes = (f, h, w)
    angs = []
    for i, (d, n) in enumerate(zip(axes_dim, sizes)):
        fr = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64)[: d // 2] / d))
        a = torch.outer(torch.arange(n, dtype=torch.float64), fr)
        shape = [1, 1, 1, d // 2]
        shape[i] = n
        angs.append(a.view(shape).expand(f, h, w, d // 2))
    ang = torch.cat(angs, dim=-1).reshape(f * h * w, -1)
    tab = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()
    return tab.to(device) if device is not None else tab


class HeadNorm(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))


class FeedForward(nn.Module):
    """diffusers-style ``net.0.proj`` / ``net.2`` MLP; TP shards the hidden width."""

    def __init__(self, dim, mult, tp: TPContext, act="gelu"):
        super().__init__()
        inner = int(dim * mult)
        self.act = act
        self.net = nn.ModuleList([nn.Module(), nn.Identity(), RowParallelLinear(inner, dim, tp)])
        self.net[0].proj = ColumnParallelLinear(dim, inner, tp)

    def forward(self, x_rows):
        h = self.net[0].proj(x_rows, act=self.act)
        return self.net[2](h)


# ------------------------------------------------------------------------------ token refiner
class RefinerAttention(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads = heads
        self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
        self.to_out = nn.ModuleList([nn.Linear(dim, dim)])

    def forward(self, x, mask):
        B, T, C = x.shape
        q, k, v = (l(x).view(B, T, self.heads, -1).transpose(1, 2) for l in (self.to_q, self.to_k, self.to_v))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.to_out[0](o.transpose(1, 2).reshape(B, T, C))


class RefinerFF(nn.Module):
    def __init__(self, dim, mult):
        super().__init__()
        self.net = nn.ModuleList([nn.Module(), nn.Identity(), nn.Linear(int(dim * mult), dim)])
        self.net[0].proj = nn.Linear(dim, int(dim * mult))

    def forward(self, x):
        return self.net[2](F.silu(self.net[0].proj(x)))


class RefinerBlock(nn.Module):
    def __init__(self, dim, heads, mult):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = RefinerAttention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.ff = RefinerFF(dim, mult)
        self.norm_out = nn.Module()
        self.norm_out.linear = nn.Linear(dim, 2 * dim)

    def forward(self, x, temb, mask):
        a = self.attn(self.norm1(x), mask)
        g = self.norm_out.linear(F.silu(temb)).to(x.dtype)
        g_msa, g_mlp = g.chunk(2, dim=1)
        x = x + a * g_msa.unsqueeze(1)
        return x + self.ff(self.norm2(x)) * g_mlp.unsqueeze(1)


class TokenRefiner(nn.Module):
    """Text-stream pre-processor (small: <= 256 tokens); plain PyTorch modules."""

    def __init__(self, cfg: HunyuanConfig):
        super().__init__()
        dim = cfg.hidden_size
        self.time_text_embed = CombinedEmbeddings(dim, cfg.text_embed_dim, guidance=False)
        self.proj_in = nn.Linear(cfg.text_embed_dim, dim)
        self.token_refiner = nn.Module()
        self.token_refiner.refiner_blocks = nn.ModuleList(
            [RefinerBlock(dim, cfg.num_attention_heads, cfg.mlp_ratio) for _ in range(cfg.num_refiner_layers)])

    def forward(self, text, timestep, attn_mask):
        if attn_mask is None:
            pooled = text.float().mean(dim=1)
        else:
            m = attn_mask.float().unsqueeze(-1)
            pooled = (text.float() * m).sum(1) / m.sum(1)
        temb = self.time_text_embed(timestep, pooled)
        x = self.proj_in(text)
        mask = None
        if attn_mask is not None:
            B, T = attn_mask.shape
            m1 = attn_mask.bool().view(B, 1, 1, T).expand(B, 1, T, T)
            mask = (m1 & m1.transpose(2, 3)).clone()
            mask[:, :, :, 0] = True
        for blk in self.token_refiner.refiner_blocks:
            x = blk(x, temb.to(x.dtype), mask)
        return x


# ------------------------------------------------------------------------------ joint attention
class _GatherHeads(torch.autograd.Function):
    """[B, T, Hl, D] -> [B, T, P*Hl, D] (rank order); backward sums over ranks and keeps our slice."""

    @staticmethod
    def forward(ctx, x, group, P, rank):
        ctx.meta = (group, P, rank, x.shape[2])
        parts = [torch.empty_like(x) for _ in range(P)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=2)

    @staticmethod
    def backward(ctx, g):
        group, P, rank, Hl = ctx.meta
        g = g.contiguous().clone()
        dist.all_reduce(g, group=group)
        return g[:, :, rank * Hl:(rank + 1) * Hl].contiguous(), None, None, None


def joint_attention(qv, kv, vv, qt, kt, vt, cp: Optional[UlyssesContext], text_lens: Optional[torch.Tensor]):
    """Video q/k/v local [B, S_l, H, D], text q/k/v replicated [B, T, H, D]. Returns (ov [B,S_l,H,D],
    ot [B,T,H,D]) of attention over the concatenated sequence with padded text keys masked."""
    B, S_l, H, D = qv.shape
    T = qt.shape[1]
    P = cp.size if cp is not None else 1
    if P > 1:
        assert H % P == 0, "heads must divide by the context-parallel size"
        Hl = H // P
        qv, kv, vv = (_SeqToHead.apply(t.contiguous(), cp.group, P) for t in (qv, kv, vv))
        qt, kt, vt = (t[:, :, cp.rank * Hl:(cp.rank + 1) * Hl] for t in (qt, kt, vt))
    S = qv.shape[1]
    q = torch.cat([qv, qt], dim=1)
    k = torch.cat([kv, kt], dim=1)
    v = torch.cat([vv, vt], dim=1)
    kv_lens = None
    if text_lens is not None:
        kv_lens = (text_lens.to(torch.int32) + S).to(q.device)
    o = ops.attention(q, k, v, None, kv_lens)
    ov, ot = o[:, :S], o[:, S:]
    if P > 1:
        ov = _HeadToSeq.apply(ov.contiguous(), cp.group, P)
        ot = _GatherHeads.apply(ot.contiguous(), cp.group, P, cp.rank)
    return ov, ot


class HunyuanAttention(nn.Module):
    """q/k/v (+ optional text-stream add_* projections) with per-head RMSNorm; diffusers key names."""

    def __init__(self, cfg: HunyuanConfig, tp: TPContext, dual: bool):
        super().__init__()
        C, D = cfg.hidden_size, cfg.attention_head_dim
        self.tp, self.D, self.eps, self.dual = tp, D, cfg.eps, dual
        self.heads_local = cfg.num_attention_heads // tp.size
        # q / k / v as one column-parallel GEMM (one all-gather -> GEMM under TP); checkpoints keep to_q / to_k / to_v
        self.to_qkv = FusedColumnParallel(C, C, ("to_q", "to_k", "to_v"), tp)
        FusedColumnParallel.install_state_hooks(self, "to_qkv")
        self.norm_q, self.norm_k = HeadNorm(D), HeadNorm(D)
        if dual:
            self.to_out = nn.ModuleList([RowParallelLinear(C, C, tp)])
            self.add_qkv_proj = FusedColumnParallel(C, C, ("add_q_proj", "add_k_proj", "add_v_proj"), tp)
            FusedColumnParallel.install_state_hooks(self, "add_qkv_proj")
            self.norm_added_q, self.norm_added_k = HeadNorm(D), HeadNorm(D)
            self.to_add_out = RowParallelLinear(C, C, tp)

    def qkv(self, x_rows, freqs, text: bool, B: int):
        """x_rows: TP-row-sharded [rows/T, C]. Returns q, k, v as [B, tokens, H_local, D]."""
        use_add = text and self.dual
        proj = self.add_qkv_proj if use_add else self.to_qkv
        nq, nk = (self.norm_added_q, self.norm_added_k) if use_add else (self.norm_q, self.norm_k)
        q_pre, k_pre, v = proj.split(proj(x_rows))
        q = ops.rmsnorm_rope(q_pre, nq.weight, freqs, self.D, True, self.eps)
        k = ops.rmsnorm_rope(k_pre, nk.weight, freqs, self.D, True, self.eps)
        n = q_pre.shape[0] // B
        return tuple(t.reshape(B, n, self.heads_local, self.D) for t in (q, k, v))

    def attend(self, hv, ht, freqs, B, cp, text_lens):
        """Joint attention of the (modulated) video rows ``hv`` and text rows ``ht``; returns the attention outputs
        (video [B, S_l, H_local, D], text [B, T, H_local, D]).  On one NVLink box the context-parallel exchanges of
        the video q / k / v and of the output are stores of the norm and attention kernels into peer memory
        (``parallel.fused_ulysses``); otherwise all-to-alls."""
        fu = cp.fused if (cp is not None and cp.size > 1) else None
        if (fu is not None and hv.is_cuda and fu.supports(self.heads_local, self.D)
                and self.heads_local % cp.size == 0):
            q_pre, k_pre, v = self.to_qkv.split(self.to_qkv(hv))
            qt, kt, vt = self.qkv(ht, None, True, B)
            S_l = q_pre.shape[0] // B
            ov, ot = fu.joint_attention(q_pre, k_pre, v, self.norm_q.weight, self.norm_k.weight, freqs, qt, kt, vt,
                                        text_lens, B, S_l, self.heads_local, self.D, self.eps)
            ot = _GatherHeads.apply(ot.contiguous(), cp.group, cp.size, cp.rank)
            return ov.view(B, S_l, self.heads_local, self.D), ot
        qv, kv, vv = self.qkv(hv, freqs, False, B)
        qt, kt, vt = self.qkv(ht, None, True, B)
        return joint_attention(qv, kv, vv, qt, kt, vt, cp, text_lens)


def _gated_residual(y_rows, residual, gate, rows_per_batch):
    """residual + gate[batch] * y for row matrices (used where the projection ends in a reduce-scatter)."""
    g = gate.repeat_interleave(rows_per_batch, dim=0)[: y_rows.shape[0]]
    return (residual.float() + g * y_rows.float()).to(residual.dtype)


def _project_out(lin: RowParallelLinear, a_rows, residual, gate, rows_per_batch):
    if lin.tp.size == 1 and a_rows.is_cuda:
        return ops.linear_residual(a_rows, lin.weight, lin.bias, residual, gate, rows_per_batch)
    return _gated_residual(lin(a_rows), residual, gate, rows_per_batch)


class AdaNormZero(nn.Module):
    def __init__(self, dim, n):
        super().__init__()
        self.linear = nn.Linear(dim, n * dim)
        self.n = n

    def forward(self, temb):
        e = F.linear(F.silu(temb.float()), self.linear.weight.float(), self.linear.bias.float())
        return e.unflatten(1, (self.n, -1))  # [B, n, C] fp32


class DualStreamBlock(nn.Module):
    def __init__(self, cfg: HunyuanConfig, tp: TPContext):
        super().__init__()
        C = cfg.hidden_size
        self.eps = cfg.eps
        self.norm1, self.norm1_context = AdaNormZero(C, 6), AdaNormZero(C, 6)
        self.attn = HunyuanAttention(cfg, tp, dual=True)
        self.ff = FeedForward(C, cfg.mlp_ratio, tp)
        self.ff_context = FeedForward(C, cfg.mlp_ratio, tp)

    def forward(self, xv, xt, temb, freqs, B, cp, text_lens):
        rv, rt = xv.shape[0] // B, xt.shape[0] // B
        ev, et = self.norm1(temb), self.norm1_context(temb)
        # each norm hands its input back for the residual branch: the residual's gradient is then added inside
        # the norm's backward kernel instead of by a separate add
        hv, xv = ops.adaln_res(xv, ev[:, 1], ev[:, 0], rv, self.eps)
        ht, xt = ops.adaln_res(xt, et[:, 1], et[:, 0], rt, self.eps)
        ov, ot = self.attn.attend(hv, ht, freqs, B, cp, text_lens)
        xv = _project_out(self.attn.to_out[0], ov.reshape(-1, ov.shape[2] * ov.shape[3]), xv, ev[:, 2], rv)
        xt = _project_out(self.attn.to_add_out, ot.reshape(-1, ot.shape[2] * ot.shape[3]), xt, et[:, 2], rt)
        hv, xv = ops.adaln_res(xv, ev[:, 4], ev[:, 3], rv, self.eps)
        ht, xt = ops.adaln_res(xt, et[:, 4], et[:, 3], rt, self.eps)
        xv = _gated_residual(self.ff(hv), xv, ev[:, 5], rv)
        xt = _gated_residual(self.ff_context(ht), xt, et[:, 5], rt)
        return xv, xt


class SingleProjOut(RowParallelLinear):
    """proj_out of the single-stream block: input columns are [attention C | mlp 4C]; under TP each
    group is sharded separately (``col_groups``)."""

    def __init__(self, dim, mlp_dim, tp):
        super().__init__(dim + mlp_dim, dim, tp)
        self.col_groups = (dim, mlp_dim)


class SingleStreamBlock(nn.Module):
    def __init__(self, cfg: HunyuanConfig, tp: TPContext):
        super().__init__()
        C = cfg.hidden_size
        mlp = int(C * cfg.mlp_ratio)
        self.eps = cfg.eps
        self.attn = HunyuanAttention(cfg, tp, dual=False)
        self.norm = AdaNormZero(C, 3)
        self.proj_mlp = ColumnParallelLinear(C, mlp, tp)
        self.proj_out = SingleProjOut(C, mlp, tp)

    def forward(self, xv, xt, temb, freqs, B, cp, text_lens):
        rv, rt = xv.shape[0] // B, xt.shape[0] // B
        e = self.norm(temb)  # shift, scale, gate
        hv, xv = ops.adaln_res(xv, e[:, 1], e[:, 0], rv, self.eps)
        ht, xt = ops.adaln_res(xt, e[:, 1], e[:, 0], rt, self.eps)
        ov, ot = self.attn.attend(hv, ht, freqs, B, cp, text_lens)
        mv = self.proj_mlp(hv, act="gelu")
        mt = self.proj_mlp(ht, act="gelu")
        cv = torch.cat([ov.reshape(mv.shape[0], -1), mv], dim=1)
        ct = torch.cat([ot.reshape(mt.shape[0], -1), mt], dim=1)
        xv = _project_out(self.proj_out, cv, xv, e[:, 2], rv)
        xt = _project_out(self.proj_out, ct, xt, e[:, 2], rt)
        return xv, xt


class _PairBlock(nn.Module):
    """Adapts a (video, text) block to the single-tensor block-stack runner by packing both streams."""

    def __init__(self, blk):
        super().__init__()
        self.blk = blk

    def forward(self, packed, n_video_rows, temb, freqs, B, cp, text_lens):
        xv, xt = packed[:n_video_rows], packed[n_video_rows:]
        xv, xt = self.blk(xv, xt, temb, freqs, B, cp, text_lens)
        return torch.cat([xv, xt], dim=0)


# ------------------------------------------------------------------------------ model
@MODELS.register("HunyuanVideoModel")
class HunyuanVideoModel(nn.Module):
    """forward(hidden_states, timestep, encoder_hidden_states, encoder_attention_mask,
    pooled_projections, guidance) -> velocity prediction [B, C_out, F, H, W]
    (teletron/models/hunyuan/parallel_model.py:272-390)."""

    def __init__(self, cfg: HunyuanConfig, cp: Optional[UlyssesContext] = None, tp: Optional[TPContext] = None):
        super().__init__()
        self.cfg, self.cp = cfg, cp
        self.tp = tp or TPContext()
        C = cfg.hidden_size
        p, pt = cfg.patch_size, cfg.patch_size_t
        self.x_embedder = nn.Module()
        self.x_embedder.proj = nn.Conv3d(cfg.in_channels, C, kernel_size=(pt, p, p), stride=(pt, p, p))
        self.context_embedder = TokenRefiner(cfg)
        self.time_text_embed = CombinedEmbeddings(C, cfg.pooled_projection_dim, cfg.guidance_embeds)
        self.transformer_blocks = nn.ModuleList([DualStreamBlock(cfg, self.tp) for _ in range(cfg.num_layers)])
        self.single_transformer_blocks = nn.ModuleList(
            [SingleStreamBlock(cfg, self.tp) for _ in range(cfg.num_single_layers)])
        self.norm_out = nn.Module()
        self.norm_out.linear = nn.Linear(C, 2 * C)
        self.proj_out = nn.Linear(C, pt * p * p * cfg.out_channels)
        self._rope_cache = {}
        self.return_local_shard = False

    def rope(self, grid, device):
        key = (tuple(grid), str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = hunyuan_rope_table(self.cfg.rope_axes_dim, grid, self.cfg.rope_theta, device)
        return self._rope_cache[key]

    def patchify(self, x):
        B, Cin, Fr, Hh, Ww = x.shape
        p, pt = self.cfg.patch_size, self.cfg.patch_size_t
        f, h, w = Fr // pt, Hh // p, Ww // p
        t = x.reshape(B, Cin, f, pt, h, p, w, p).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return t.reshape(B * f * h * w, Cin * pt * p * p), (f, h, w)

    def unpatchify(self, x, grid):
        """[B, S, C_out*pt*p*p] with per-token order (c, pt, p, p) -> [B, C_out, F, H, W]."""
        f, h, w = grid
        p, pt = self.cfg.patch_size, self.cfg.patch_size_t
        B = x.shape[0]
        x = x.reshape(B, f, h, w, self.cfg.out_channels, pt, p, p).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return x.reshape(B, self.cfg.out_channels, f * pt, h * p, w * p)

    def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_attention_mask=None,
                pooled_projections=None, guidance=None, **_):
        cfg = self.cfg
        dt = self.proj_out.weight.dtype
        B = hidden_states.shape[0]
        if self.tp.size > 1:
            assert B == 1, "tensor parallelism with sequence-sharded activations expects micro-batch 1"
        dev = hidden_states.device
        timestep = timestep.to(dev).float().reshape(-1).expand(B)
        temb = self.time_text_embed(timestep, pooled_projections.to(dev).float(),
                                    guidance.to(dev).float().reshape(-1).expand(B) if guidance is not None else None)
        patches, grid = self.patchify(hidden_states.to(dt))
        S = grid[0] * grid[1] * grid[2]
        C = cfg.hidden_size
        xv = ops.linear(patches.contiguous(), self.x_embedder.proj.weight.view(C, -1), self.x_embedder.proj.bias)
        xt = self.context_embedder(encoder_hidden_states.to(dt), timestep, encoder_attention_mask)
        T = xt.shape[1]
        xt = xt.reshape(B * T, C)
        text_lens = encoder_attention_mask.sum(dim=1) if encoder_attention_mask is not None else None
        freqs = self.rope(grid, dev)
        cp = self.cp if (self.cp is not None and self.cp.size > 1) else None
        if cp is not None:
            assert S % cp.size == 0, "video tokens must divide by the context-parallel size"
            xv = cp.split_tokens(xv.view(B, S, C)).reshape(-1, C)
            freqs = cp.split_rows(freqs)
            fu = cp.fused
            if fu is not None and xv.is_cuda:
                # symmetric slab for the joint q / k / v (head layout) and the video output of every live layer
                alive = cfg.num_layers + cfg.num_single_layers
                if self.training and cfg.recompute_granularity == "full":
                    # checkpointed blocks give their region back at once; the others keep theirs until backward
                    k = cfg.recompute_num_layers or 0
                    if (cfg.recompute_method or "block") == "block":
                        alive = (cfg.num_layers - min(k, cfg.num_layers)
                                 + cfg.num_single_layers - min(k, cfg.num_single_layers) + 2)
                    else:
                        alive = max(k, 1) + 1
                heads_local = cfg.num_attention_heads // self.tp.size
                per_layer = (3 * B * (S + (T + 7) // 8 * 8) * (heads_local // cp.size) * cfg.attention_head_dim
                             + B * (S // cp.size) * heads_local * cfg.attention_head_dim + 4 * 128)
                fu.begin_microbatch(int(per_layer * alive * 1.02) + 512)
        if self.tp.size > 1:  # sequence-sharded activations between tensor-parallel regions
            xv, xt = self.tp.split_rows(xv), self.tp.split_rows(xt)
            freqs_attn = freqs  # attention sees the TP-gathered rows
        else:
            freqs_attn = freqs
        n_v = xv.shape[0]
        packed = torch.cat([xv, xt], dim=0)
        extra = (n_v, temb, freqs_attn, B, cp, text_lens)
        packed = rc.run_blocks([_PairBlock(b) for b in self.transformer_blocks], packed, extra, cfg, self.training)
        packed = rc.run_blocks([_PairBlock(b) for b in self.single_transformer_blocks], packed, extra, cfg, self.training)
        xv = packed[:n_v]
        e = F.linear(F.silu(temb), self.norm_out.linear.weight.float(), self.norm_out.linear.bias.float())
        e = e.unflatten(1, (2, C))  # scale, shift
        rows_per_batch = xv.shape[0] // B
        h = ops.adaln(xv.contiguous(), e[:, 0], e[:, 1], rows_per_batch, cfg.eps)
        out = ops.linear(h, self.proj_out.weight, self.proj_out.bias)
        if self.tp.size > 1:
            out = self.tp.gather_rows_for_output(out)
        out = out.view(B, -1, out.shape[-1])
        if cp is not None:
            if self.return_local_shard:
                return out
            out = cp.gather_tokens(out, S)
        return self.unpatchify(out, grid)

    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        return self.state_dict(prefix=prefix, keep_vars=keep_vars)

    def set_input_tensor(self, input_tensor):
        return None


def hunyuan_config_from_args(a) -> HunyuanConfig:
    if isinstance(a, HunyuanConfig):
        return a
    kw = dict(HUNYUAN_PRESETS.get(getattr(a, "model_preset", None) or "hunyuanvideo-13b-t2v"))
    if getattr(a, "hidden_size", None):
        kw["hidden_size"] = a.hidden_size
    if getattr(a, "num_attention_heads", None):
        kw["num_attention_heads"] = a.num_attention_heads
    if getattr(a, "num_layers", None):
        kw["num_layers"] = a.num_layers
    for f in ("num_single_layers", "num_refiner_layers", "text_embed_dim", "pooled_projection_dim"):
        if getattr(a, f, None):
            kw[f] = getattr(a, f)
    if getattr(a, "task_type", None) == "i2v":
        kw["in_channels"] = 33
    kw["recompute_granularity"] = getattr(a, "recompute_granularity", None)
    kw["recompute_method"] = getattr(a, "recompute_method", None) or "block"
    kw["recompute_num_layers"] = getattr(a, "recompute_num_layers", None) or 0
    kw["activation_offload"] = bool(getattr(a, "activation_offload", False))
    return HunyuanConfig(**kw)


@MODELS.register("ParallelHunyuanVideoModel")
class ParallelHunyuanVideoModel(HunyuanVideoModel):
    def __init__(self, config, cp=None, tp=None, **_):
        from ..parallel import state as mpu

        cfg = hunyuan_config_from_args(config)
        if mpu.model_parallel_is_initialized():
            if cp is None and mpu.get_context_parallel_world_size() > 1:
                cp = UlyssesContext(mpu.get_context_parallel_group(), mpu.get_context_parallel_world_size(),
                                    mpu.get_context_parallel_rank())
            if tp is None and mpu.get_tensor_model_parallel_world_size() > 1:
                tp = TPContext(mpu.get_tensor_model_parallel_group(), mpu.get_tensor_model_parallel_world_size(),
                               mpu.get_tensor_model_parallel_rank())
        super().__init__(cfg, cp, tp)
