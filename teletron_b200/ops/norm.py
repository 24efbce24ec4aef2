"""Row normalisation ops: AdaLN (LayerNorm + timestep modulation), affine LayerNorm and
RMSNorm fused with rotary embedding — csrc/norm.cu.

All tensors are 2-D ``[rows, C]`` bf16 (row stride free); modulation vectors are fp32
``[batch, C]`` views (row stride free), row ``r`` uses modulation row ``r // rows_per_batch``.
Each op has a differentiable PyTorch reference (``*_ref``) which is also the CPU path.
They replace teletron_op/fused_adaln, teletron_op/fused_rmsnorm and the modulate / rope_apply
ATen chains of the reference (teletron/models/wan/wan_model.py:77-78,105-124).
"""
from __future__ import annotations

import torch

from . import _lib

_CHUNKS_TARGET = 592  # CTAs for column-reduction kernels (4 per SM)


def _chunks(rows_per_batch: int, batch: int) -> int:
    return max(1, min(rows_per_batch, _CHUNKS_TARGET // max(batch, 1)))


# --------------------------------------------------------------------------- AdaLN
def adaln_ref(x, scale, shift, rows_per_batch, eps=1e-6, plus_one=True):
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    xh = (xf - mean) * torch.rsqrt(var + eps)
    rows = x.shape[0]

    def expand(m):
        return m.float().repeat_interleave(rows_per_batch, dim=0)[:rows]

    if scale is not None:
        xh = xh * ((1.0 + expand(scale)) if plus_one else expand(scale))
    if shift is not None:
        xh = xh + expand(shift)
    return xh.to(x.dtype)


class _AdaLN(torch.autograd.Function):
    """``with_res``: also return x itself as a second output (an alias) for the residual connection, so that
    the residual's gradient arrives here and is added inside the backward kernel (no separate add kernel)."""

    @staticmethod
    def forward(ctx, x, scale, shift, rows_per_batch, eps, plus_one, with_res=False):
        rows, C = x.shape
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1
        for m in (scale, shift):
            if m is not None:
                assert m.dtype == torch.float32 and m.dim() == 2 and m.stride(1) == 1 and m.shape[1] == C
        batch = (rows + rows_per_batch - 1) // rows_per_batch
        y = torch.empty((rows, C), dtype=torch.bfloat16, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        ref = scale if scale is not None else shift
        mod_ld = ref.stride(0) if ref is not None else 0
        if scale is not None and shift is not None:
            assert scale.stride(0) == shift.stride(0)
        rc = _lib.lib().tt_adaln_fwd(
            _lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(y), _lib.c_ll(C), _lib.ptr(scale), _lib.ptr(shift),
            _lib.c_ll(mod_ld), _lib.c_int(int(plus_one)), _lib.c_int(rows), _lib.c_int(C),
            _lib.c_int(rows_per_batch), _lib.c_float(eps), _lib.ptr(mean), _lib.ptr(rstd), _lib.stream())
        _lib.check(rc, "tt_adaln_fwd")
        ctx.save_for_backward(x, mean, rstd, scale)
        ctx.meta = (rows_per_batch, plus_one, batch, mod_ld, shift is not None)
        if with_res:
            return y, x.view_as(x)
        return y

    @staticmethod
    def backward(ctx, dy, dres=None):
        x, mean, rstd, scale = ctx.saved_tensors
        rows_per_batch, plus_one, batch, mod_ld, has_shift = ctx.meta
        rows, C = x.shape
        assert rows == batch * rows_per_batch, "adaln backward needs rows == batch * rows_per_batch"
        if dy is None:  # only the residual alias was used
            return dres, None, None, None, None, None, None
        if dy.stride(1) != 1:
            dy = dy.contiguous()
        if dres is not None and (dres.dtype != torch.bfloat16 or dres.stride(1) != 1):
            dres = dres.to(torch.bfloat16).contiguous()
        dx = torch.empty((rows, C), dtype=torch.bfloat16, device=x.device)
        want_mod = (scale is not None and ctx.needs_input_grad[1]) or (has_shift and ctx.needs_input_grad[2])
        chunks = _chunks(rows_per_batch, batch)
        partial = dmul = dadd = None
        if want_mod:
            partial = torch.empty((batch, chunks, 2, C), dtype=torch.float32, device=x.device)
            dmul = torch.empty((batch, C), dtype=torch.float32, device=x.device) if scale is not None else None
            dadd = torch.empty((batch, C), dtype=torch.float32, device=x.device) if has_shift else None
        rc = _lib.lib().tt_adaln_bwd(
            _lib.ptr(dy), _lib.c_ll(dy.stride(0)), _lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(mean),
            _lib.ptr(rstd), _lib.ptr(scale), _lib.c_ll(mod_ld), _lib.c_int(int(plus_one)), _lib.ptr(dx),
            _lib.c_ll(C), _lib.ptr(dres), _lib.c_ll(dres.stride(0) if dres is not None else 0), _lib.ptr(partial),
            _lib.c_int(chunks),
            _lib.ptr(dmul), _lib.ptr(dadd), _lib.c_int(0), _lib.c_int(batch), _lib.c_int(rows_per_batch),
            _lib.c_int(C), _lib.stream())
        _lib.check(rc, "tt_adaln_bwd")
        return dx, dmul, dadd, None, None, None, None


def adaln(x, scale, shift, rows_per_batch, eps=1e-6, plus_one=True):
    """LayerNorm(no affine)(x) * (1 + scale) + shift, fp32 statistics."""
    if not x.is_cuda:
        return adaln_ref(x, scale, shift, rows_per_batch, eps, plus_one)
    return _AdaLN.apply(x, scale, shift, rows_per_batch, eps, plus_one)


def adaln_res(x, scale, shift, rows_per_batch, eps=1e-6, plus_one=True):
    """(adaln(x), x): the second value is x for the residual branch; its gradient is added to the norm's input
    gradient inside the backward kernel."""
    if not x.is_cuda:
        return adaln_ref(x, scale, shift, rows_per_batch, eps, plus_one), x
    return _AdaLN.apply(x, scale, shift, rows_per_batch, eps, plus_one, True)


def layernorm_affine(x, weight, bias, eps=1e-6, with_res=False):
    """nn.LayerNorm with affine parameters (Wan ``norm3``) through the AdaLN kernel."""
    rows = x.shape[0]
    w = weight.float().unsqueeze(0) if weight is not None else None
    b = bias.float().unsqueeze(0) if bias is not None else None
    if with_res:
        return adaln_res(x, w, b, rows, eps, plus_one=False)
    return adaln(x, w, b, rows, eps, plus_one=False)


# --------------------------------------------------------------------------- RMSNorm + RoPE
def rope_ref(x, freqs, D):
    """x [rows, C] ; freqs [S, D/2, 2] (cos, sin); row r uses freqs[r % S]. Interleaved pairs."""
    rows, C = x.shape
    S = freqs.shape[0]
    H = C // D
    xf = x.float().reshape(rows, H, D // 2, 2)
    idx = torch.arange(rows, device=x.device) % S
    cs = freqs.to(x.device)[idx].unsqueeze(1)  # [rows,1,D/2,2]
    c, s = cs[..., 0], cs[..., 1]
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack((a * c - b * s, a * s + b * c), dim=-1)
    return out.reshape(rows, C)


def rmsnorm_rope_ref(x, weight, freqs, D, per_head=False, eps=1e-6):
    rows, C = x.shape
    xf = x.float()
    if weight is not None:
        if per_head:
            xh = xf.reshape(rows, C // D, D)
            xh = xh * torch.rsqrt(xh.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
            xf = xh.reshape(rows, C)
        else:
            xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    if freqs is not None:
        xf = rope_ref(xf, freqs, D)
    return xf.to(x.dtype)


def rmsrope_fwd_raw(x, wf, freqs, D, per_head=False, eps=1e-6):
    """rope(rmsnorm(x) * wf) without autograd: returns (y bf16 [rows, C], rstd fp32 or None). ``x`` may be a
    column slice of a wider tensor (row stride > C)."""
    rows, C = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    if freqs is not None:
        assert freqs.dtype == torch.float32 and freqs.is_contiguous() and freqs.shape[1:] == (D // 2, 2)
    y = torch.empty((rows, C), dtype=torch.bfloat16, device=x.device)
    rstd = None
    if wf is not None:
        rstd = torch.empty(rows * (C // D if per_head else 1), dtype=torch.float32, device=x.device)
    rc = _lib.lib().tt_rmsrope_fwd(
        _lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(y), _lib.c_ll(C), _lib.ptr(wf), _lib.ptr(freqs),
        _lib.c_int(freqs.shape[0] if freqs is not None else 1), _lib.ptr(rstd), _lib.c_int(rows),
        _lib.c_int(C), _lib.c_int(D), _lib.c_int(int(per_head)), _lib.c_float(eps), _lib.stream())
    _lib.check(rc, "tt_rmsrope_fwd")
    return y, rstd


class _RmsRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, freqs, D, per_head, eps):
        wf = weight.float().contiguous() if weight is not None else None
        y, rstd = rmsrope_fwd_raw(x, wf, freqs, D, per_head, eps)
        ctx.save_for_backward(x, wf, freqs, rstd)
        ctx.meta = (D, per_head, weight.dtype if weight is not None else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wf, freqs, rstd = ctx.saved_tensors
        D, per_head, wdtype = ctx.meta
        dx, dw = rmsrope_bwd_raw(dy, x, wf, freqs, rstd, D, per_head)
        return dx, (dw.to(wdtype) if dw is not None else None), None, None, None, None


def rmsrope_bwd_raw(dy, x, wf, freqs, rstd, D, per_head=False, out=None):
    """Backward of rope(rmsnorm(x) * w) from the saved input and rstd: returns (dx bf16, dw fp32 or None).
    ``out``: optional [rows, C] view (any row stride) that receives dx."""
    rows, C = x.shape
    if dy.stride(1) != 1:
        dy = dy.contiguous()
    dx = out if out is not None else torch.empty((rows, C), dtype=torch.bfloat16, device=x.device)
    assert dx.shape == (rows, C) and dx.stride(1) == 1 and dx.dtype == torch.bfloat16
    L = _lib.lib()
    partial = None
    ctas = L.tt_rmsrope_bwd_ctas(_lib.c_int(rows))
    if wf is not None:
        partial = torch.empty((ctas, C), dtype=torch.float32, device=x.device)
    rc = L.tt_rmsrope_bwd(
        _lib.ptr(dy), _lib.c_ll(dy.stride(0)), _lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(dx),
        _lib.c_ll(dx.stride(0)), _lib.ptr(wf), _lib.ptr(freqs), _lib.c_int(freqs.shape[0] if freqs is not None else 1),
        _lib.ptr(rstd), _lib.ptr(partial), _lib.c_int(rows), _lib.c_int(C), _lib.c_int(D),
        _lib.c_int(int(per_head)), _lib.stream())
    _lib.check(rc, "tt_rmsrope_bwd")
    dw = None
    if wf is not None:
        dwf = torch.empty((1, C), dtype=torch.float32, device=x.device)
        rc = L.tt_colsum_partials(_lib.ptr(partial), _lib.ptr(dwf), _lib.c_int(1), _lib.c_int(ctas),
                                  _lib.c_int(C), _lib.c_int(0), _lib.stream())
        _lib.check(rc, "tt_colsum_partials")
        dw = dwf.view(C // D, D).sum(0) if per_head else dwf.view(C)
    return dx, dw


def rmsnorm_rope(x, weight, freqs, D, per_head=False, eps=1e-6):
    """rope(rmsnorm(x) * weight); weight None skips the norm, freqs None skips the rotation."""
    if not x.is_cuda:
        return rmsnorm_rope_ref(x, weight, freqs, D, per_head, eps)
    return _RmsRope.apply(x, weight, freqs, D, per_head, eps)
