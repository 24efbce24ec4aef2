"""Flash attention (non-causal, head_dim 128) on tcgen05 — csrc/attn_fwd.cu, csrc/attn_bwd.cu.

Tensors are ``[B, S, H, D]`` views whose last two dims are dense (``stride(-1) == 1``,
``stride(-2) == D``); token and batch strides are free, so q/k/v can be column slices of
a fused QKV projection.  ``attention_ref`` is the fp32 PyTorch statement (also the CPU
path).  Replaces flash_attn / SDPA of the reference
(teletron/core/context_parallel/context_parallel_mixin.py:107-114).
"""
from __future__ import annotations

import math

import torch

from . import _lib


def attention_ref(q, k, v, scale=None, kv_lens=None):
    """fp32 reference: q [B,Sq,H,D], k/v [B,Skv,H,D] -> (o [B,Sq,H,D] in q.dtype, lse [B,H,Sq] fp32)."""
    B, Sq, H, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if kv_lens is not None:
        idx = torch.arange(k.shape[1], device=q.device)[None, None, None, :]
        s = s.masked_fill(idx >= kv_lens.to(q.device)[:, None, None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vf)
    return o.permute(0, 2, 1, 3).to(q.dtype), lse


def _check_layout(t: torch.Tensor, name: str):
    assert t.dim() == 4 and t.stride(3) == 1 and t.stride(2) == t.shape[3], (
        f"{name}: expected [B,S,H,D] with dense (H,D), got strides {t.stride()}")


def attention_fwd(q, k, v, scale=None, kv_lens=None):
    """Returns (o [B,Sq,H,D] bf16 contiguous, lse [B,H,Sq] fp32)."""
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        return attention_ref(q, k, v, scale, kv_lens)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_layout(t, n)
        assert t.dtype == torch.bfloat16
    o = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    if kv_lens is not None:
        kv_lens = kv_lens.to(device=q.device, dtype=torch.int32).contiguous()
    L = _lib.lib()
    rc = L.tt_attn_fwd(
        _lib.ptr(q), _lib.c_ll(q.stride(1)), _lib.c_ll(q.stride(0)),
        _lib.ptr(k), _lib.c_ll(k.stride(1)), _lib.c_ll(k.stride(0)),
        _lib.ptr(v), _lib.c_ll(v.stride(1)), _lib.c_ll(v.stride(0)),
        _lib.ptr(o), _lib.c_ll(o.stride(1)), _lib.c_ll(o.stride(0)),
        _lib.ptr(lse), _lib.ptr(kv_lens), _lib.c_int(B), _lib.c_int(H), _lib.c_int(Sq),
        _lib.c_int(Skv), _lib.c_int(D), _lib.c_float(scale), _lib.ptr(_lib.status_word(q.device)),
        _lib.stream())
    _lib.check(rc, "tt_attn_fwd")
    return o, lse


def attention_bwd(q, k, v, o, lse, dout, scale=None, kv_lens=None):
    """Gradients (dq, dk, dv), each [B,S,H,D] bf16 contiguous."""
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (dout, "dout")):
        _check_layout(t, n)
        assert t.dtype == torch.bfloat16
    dq = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q.device)
    dk = torch.empty((B, Skv, H, D), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty((B, Skv, H, D), dtype=torch.bfloat16, device=q.device)
    L = _lib.lib()
    L.tt_attn_bwd_scratch_floats.restype = _lib.c_ll
    n_scratch = L.tt_attn_bwd_scratch_floats(_lib.c_int(B), _lib.c_int(H), _lib.c_int(Sq))
    scratch = torch.empty(n_scratch, dtype=torch.float32, device=q.device)
    if kv_lens is not None:
        kv_lens = kv_lens.to(device=q.device, dtype=torch.int32).contiguous()
    lse = lse.contiguous()
    rc = L.tt_attn_bwd(
        _lib.ptr(q), _lib.c_ll(q.stride(1)), _lib.c_ll(q.stride(0)),
        _lib.ptr(k), _lib.c_ll(k.stride(1)), _lib.c_ll(k.stride(0)),
        _lib.ptr(v), _lib.c_ll(v.stride(1)), _lib.c_ll(v.stride(0)),
        _lib.ptr(o), _lib.c_ll(o.stride(1)), _lib.c_ll(o.stride(0)),
        _lib.ptr(dout), _lib.c_ll(dout.stride(1)), _lib.c_ll(dout.stride(0)),
        _lib.ptr(lse), _lib.ptr(scratch),
        _lib.ptr(dq), _lib.c_ll(dq.stride(1)), _lib.c_ll(dq.stride(0)),
        _lib.ptr(dk), _lib.c_ll(dk.stride(1)), _lib.c_ll(dk.stride(0)),
        _lib.ptr(dv), _lib.c_ll(dv.stride(1)), _lib.c_ll(dv.stride(0)),
        _lib.ptr(kv_lens), _lib.c_int(B), _lib.c_int(H), _lib.c_int(Sq), _lib.c_int(Skv),
        _lib.c_int(D), _lib.c_float(scale), _lib.ptr(_lib.status_word(q.device)), _lib.stream())
    _lib.check(rc, "tt_attn_bwd")
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, kv_lens):
        o, lse = attention_fwd(q, k, v, scale, kv_lens)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        ctx.kv_lens = kv_lens
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        if dout.stride(3) != 1 or dout.stride(2) != dout.shape[3]:
            dout = dout.contiguous()
        dq, dk, dv = attention_bwd(q, k, v, o, lse, dout, ctx.scale, ctx.kv_lens)
        return dq, dk, dv, None, None


def attention(q, k, v, scale=None, kv_lens=None):
    """Differentiable attention. CUDA: tcgen05 kernels; CPU: PyTorch reference (autograd)."""
    if not q.is_cuda:
        return attention_ref(q, k, v, scale, kv_lens)[0]
    return _Attention.apply(q, k, v, scale, kv_lens)
