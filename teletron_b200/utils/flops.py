"""Work and memory estimates: training FLOPs of the Wan DiT, parameter / optimizer memory per rank
and a device memory report (teletron/train/utils.py:40-213, teletron/utils/aux_func.py:803-828)."""
from __future__ import annotations

import torch


def wan_flops_per_sample(cfg, tokens: int, text_tokens: int = 512, image_tokens: int = 0, recompute: bool = False):
    """Forward+backward FLOPs of one sample (2 * MACs; backward = 2x forward for GEMMs, 2.5x for attention)."""
    C, F, L = cfg.dim, cfg.ffn_dim, cfg.num_layers
    ctx = text_tokens + image_tokens
    lin = 2 * tokens * (4 * C * C + 2 * C * C + 2 * C * F) + 2 * ctx * 2 * C * C   # self qkv+o, cross q+o, ffn; cross k,v
    attn = 4 * tokens * tokens * C + 4 * tokens * ctx * C
    fwd = L * (lin + attn)
    return fwd * ((4.0 if recompute else 3.0) * lin / (lin + attn) + (4.5 if recompute else 3.5) * attn / (lin + attn))


def theoretical_memory_gb(num_params: int, dp_cp_world: int = 1, sharded_optimizer: bool = False,
                          grad_bytes: int = 4) -> float:
    """bf16 weights + gradient buffer + fp32 master/m/v (sharded over DP x CP when requested)."""
    opt = 12.0 / (dp_cp_world if sharded_optimizer else 1)
    return num_params * (2 + grad_bytes + opt) / 2 ** 30


def memory_report(prefix: str = "") -> str:
    if not torch.cuda.is_available():
        return f"{prefix} no CUDA device"
    mb = 2 ** 20
    return (f"{prefix} memory (MB) | allocated: {torch.cuda.memory_allocated() / mb:.0f} | max allocated: "
            f"{torch.cuda.max_memory_allocated() / mb:.0f} | reserved: {torch.cuda.memory_reserved() / mb:.0f} | "
            f"max reserved: {torch.cuda.max_memory_reserved() / mb:.0f}")


def fit_activation_memory(points):
    """Least-squares line through measured ``(tokens_per_gpu, peak_GiB)`` points: returns
    ``(static_GiB, GiB_per_token)``.  With full activation recompute the peak is linear in the sequence
    length (one checkpoint per block plus one block's working set), so two runs pin it down."""
    n = len(points)
    if n < 2:
        raise ValueError("need at least two (tokens, GiB) measurements")
    mx = sum(p[0] for p in points) / n
    my = sum(p[1] for p in points) / n
    sxx = sum((p[0] - mx) ** 2 for p in points)
    if sxx == 0:
        raise ValueError("measurements must differ in sequence length")
    slope = sum((p[0] - mx) * (p[1] - my) for p in points) / sxx
    return my - slope * mx, slope


def max_trainable_frames(capacity_gib: float, static_gib: float, gib_per_token: float, height: int, width: int,
                         cp: int = 1, reserve_gib: float = 8.0) -> int:
    """Largest frame count 4k+1 whose activations fit: ``static + tokens / cp * gib_per_token`` must stay
    below ``capacity - reserve``.  ``gib_per_token`` is per token held on one GPU (Ulysses keeps 1/cp of
    the tokens, or of the heads, of every activation), ``static_gib`` the weights / gradients / optimizer
    share of that GPU.  This bounds memory only; step time grows with the square of the frame count."""
    room = capacity_gib - reserve_gib - static_gib
    if room <= 0 or gib_per_token <= 0:
        return 0
    per_latent_frame = (height // 16) * (width // 16)
    latent_frames = int(room / gib_per_token * cp) // per_latent_frame
    return 0 if latent_frames < 1 else (latent_frames - 1) * 4 + 1
