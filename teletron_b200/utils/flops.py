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


# Activation memory per token held on a GPU, calibrated on Wan2.1-1.3B runs on B200 (bf16 activations):
#   full recompute: one [C] checkpoint per block plus one block's live working set, 197 KiB per token at
#                   L = 30, C = 1536  ->  2*L*C + 36*C*2 bytes
#   no recompute:   76 GiB for 32,760 tokens at L = 30, C = 1536 (FFN 8960)  ->  about 53*C bytes per block
_WORKING_SET_WIDTHS = 36.0
_SAVED_BYTES_PER_BLOCK_WIDTH = 53.0


def activation_gib_per_token(dim: int, num_layers: int, recompute: bool = True) -> float:
    """Estimated activation memory per token on one GPU (see the calibration above); linear in the hidden size, so
    wider feed-forward ratios than Wan's 5.8x are under-counted without recompute."""
    if recompute:
        b = 2.0 * num_layers * dim + _WORKING_SET_WIDTHS * dim * 2.0
    else:
        b = _SAVED_BYTES_PER_BLOCK_WIDTH * dim * num_layers + _WORKING_SET_WIDTHS * dim * 2.0
    return b / 2 ** 30


def plan(cfg, num_params: float, height: int, width: int, frames: int, gpus: int = 1, cp: int = 1,
         recompute: bool = True, capacity_gib: float = 179.0, tflops_per_gpu: float = 850.0) -> dict:
    """Back-of-envelope plan for one configuration: tokens, FLOPs per sample, static and activation memory per GPU,
    whether it fits, the largest frame count that would, and the step time at ``tflops_per_gpu`` of executed work
    (850 is what the 14B / CP 8 step measured; the 1.3B step reaches about 1,000)."""
    tokens = ((frames - 1) // 4 + 1) * (height // 16) * (width // 16)
    static = theoretical_memory_gb(int(num_params), gpus, sharded_optimizer=gpus > 1)
    per_tok = activation_gib_per_token(cfg.dim, cfg.num_layers, recompute)
    act = tokens / cp * per_tok
    flops = wan_flops_per_sample(cfg, tokens, recompute=recompute)
    return dict(tokens=tokens, flops_per_sample=flops, static_gib=static, activation_gib=act,
                fits=static + act + 8.0 <= capacity_gib,
                max_frames=max_trainable_frames(capacity_gib, static, per_tok, height, width, cp=cp),
                seconds_per_sample=flops / (tflops_per_gpu * 1e12 * cp))
