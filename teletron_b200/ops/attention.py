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


def attention_bwd(q, k, v, o, lse, dout, scale=None, kv_lens=None, out=None):
    """Gradients (dq, dk, dv), each [B,S,H,D] bf16 contiguous, or written into the three views of ``out``
    (any token / batch strides, unit stride over H x D)."""
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (dout, "dout")):
        _check_layout(t, n)
        assert t.dtype == torch.bfloat16
    if out is not None:
        dq, dk, dv = out
        for t, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            _check_layout(t, n)
            assert t.dtype == torch.bfloat16
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    else:
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


class _SelfAttnCore(torch.autograd.Function):
    """attention(rope(rmsnorm(q) w_q), rope(rmsnorm(k) w_k), v) on the three column blocks of one [rows, 3C]
    projection output, as one autograd node: the backward kernels write dq / dk / dv straight into the three
    column blocks of one gradient tensor, so the slice-gradient zero fills, strided copies and adds that autograd
    would otherwise launch (about 1 ms per Wan2.1-1.3B block) do not exist."""

    @staticmethod
    def forward(ctx, qkv, wq, wk, freqs, batch, S, H, D, eps):
        from .norm import rmsrope_fwd_raw

        C = H * D
        assert qkv.dim() == 2 and qkv.shape == (batch * S, 3 * C) and qkv.stride(1) == 1
        wqf, wkf = wq.float().contiguous(), wk.float().contiguous()
        q, rq = rmsrope_fwd_raw(qkv[:, 0:C], wqf, freqs, D, False, eps)
        k, rk = rmsrope_fwd_raw(qkv[:, C:2 * C], wkf, freqs, D, False, eps)
        v4 = qkv[:, 2 * C:3 * C].unflatten(1, (H, D)).unflatten(0, (batch, S))
        q4, k4 = q.view(batch, S, H, D), k.view(batch, S, H, D)
        o, lse = attention_fwd(q4, k4, v4)
        ctx.save_for_backward(qkv, wqf, wkf, freqs, rq, rk, q, k, o, lse)
        ctx.meta = (batch, S, H, D, wq.dtype)
        return o.view(batch * S, C)

    @staticmethod
    def backward(ctx, do):
        from .norm import rmsrope_bwd_raw

        qkv, wqf, wkf, freqs, rq, rk, q, k, o, lse = ctx.saved_tensors
        batch, S, H, D, wdtype = ctx.meta
        C = H * D
        if do.stride(1) != 1 or do.stride(0) != C:
            do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        dqn = torch.empty((batch, S, H, D), dtype=torch.bfloat16, device=qkv.device)
        dkn = torch.empty_like(dqn)
        dv_view = dqkv[:, 2 * C:3 * C].unflatten(1, (H, D)).unflatten(0, (batch, S))
        v4 = qkv[:, 2 * C:3 * C].unflatten(1, (H, D)).unflatten(0, (batch, S))
        attention_bwd(q.view(batch, S, H, D), k.view(batch, S, H, D), v4, o, lse, do.view(batch, S, H, D),
                      out=(dqn, dkn, dv_view))
        _, dwq = rmsrope_bwd_raw(dqn.view(batch * S, C), qkv[:, 0:C], wqf, freqs, rq, D, False, out=dqkv[:, 0:C])
        _, dwk = rmsrope_bwd_raw(dkn.view(batch * S, C), qkv[:, C:2 * C], wkf, freqs, rk, D, False,
                                 out=dqkv[:, C:2 * C])
        return dqkv, dwq.to(wdtype), dwk.to(wdtype), None, None, None, None, None, None


def self_attention_core(qkv, wq, wk, freqs, batch, S, H, D, eps=1e-6):
    """Self-attention of a Wan block from the fused projection output ``qkv`` [batch * S, 3 H D] (full-row RMSNorm
    and rotary embedding on q and k): returns [batch * S, H D]."""
    if not qkv.is_cuda:
        from .norm import rmsnorm_rope

        C = H * D
        q = rmsnorm_rope(qkv[:, 0:C], wq, freqs, D, False, eps).view(batch, S, H, D)
        k = rmsnorm_rope(qkv[:, C:2 * C], wk, freqs, D, False, eps).view(batch, S, H, D)
        v = qkv[:, 2 * C:3 * C].unflatten(1, (H, D)).unflatten(0, (batch, S))
        return attention(q, k, v).reshape(batch * S, C)
    return _SelfAttnCore.apply(qkv, wq, wk, freqs, batch, S, H, D, eps)
