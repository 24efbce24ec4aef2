"""Linear layers on the tcgen05 GEMM with fused epilogues and gradient-buffer accumulation.

``linear(x, w, b, act)``            y = act(x w^T + b)            act in {None, "gelu", "silu"}
``linear_residual(x, w, b, res, gate, rows_per_gate)``
                                    y = res + gate[row // rows_per_gate] * (x w^T + b)
``ffn(x, w1, b1, w2, b2, res, gate, rows_per_gate, act)``
                                    the two composed

Backward runs dgrad with the weight read MN-major and wgrad with both operands read
MN-major (no transposes).  When the weight carries a ``main_grad`` fp32 buffer (set by
``parallel.ddp.ParamBuffer``) the weight gradient is accumulated into it inside the GEMM
epilogue and autograd receives ``None`` for it; otherwise a bf16 gradient is returned.
On CPU everything falls back to differentiable PyTorch.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import EPI_ACCUM, EPI_GATE_RES, EPI_GELU, EPI_NONE, EPI_SILU, gemm

_ACT = {None: EPI_NONE, "gelu": EPI_GELU, "silu": EPI_SILU}

_COLSUM_CHUNKS = 296


def colsum(x: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """Column sums of a bf16 [rows, C] matrix (bias gradients)."""
    if not x.is_cuda:
        return x.float().sum(0).to(out_dtype)
    rows, C = x.shape
    chunks = max(1, min(rows, _COLSUM_CHUNKS))
    partial = torch.empty((chunks, C), dtype=torch.float32, device=x.device)
    out = torch.empty(C, dtype=out_dtype, device=x.device)
    rc = _lib.lib().tt_colsum(_lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(partial), _lib.c_int(chunks),
                              _lib.ptr(out), _lib.c_int(int(out_dtype == torch.float32)), _lib.c_int(0),
                              _lib.c_int(rows), _lib.c_int(C), _lib.stream())
    _lib.check(rc, "tt_colsum")
    return out


def act_bwd(dact: torch.Tensor, pre: torch.Tensor, kind: str) -> torch.Tensor:
    rows, C = pre.shape
    out = torch.empty((rows, C), dtype=torch.bfloat16, device=pre.device)
    rc = _lib.lib().tt_act_bwd(_lib.ptr(dact), _lib.c_ll(dact.stride(0)), _lib.ptr(pre), _lib.c_ll(pre.stride(0)),
                               _lib.ptr(out), _lib.c_ll(C), _lib.c_int(rows), _lib.c_int(C),
                               _lib.c_int(0 if kind == "gelu" else 1), _lib.stream())
    _lib.check(rc, "tt_act_bwd")
    return out


def _weight_grad(dy, x, w, owner=None):
    """dW = dy^T x. Accumulates into the parameter's main_grad when present (returns None), else returns bf16.

    ``owner`` is the parameter object the forward pass was called with.  The tensor that comes back from
    ``ctx.saved_tensors`` is not always that object: inside a non-reentrant checkpoint the recompute pass hands
    back a detached alias without the parameter's Python attributes, and the gradient would silently take the
    bf16 ``.grad`` route (2 more bytes per parameter until the end of backward, and bf16 accumulation)."""
    if owner is not None:
        w = owner
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        gemm(dy, x, a_mn=True, b_mn=True, out=mg, epi=EPI_ACCUM)
        w.grad_written = True
        ready = getattr(w, "grad_ready", None)
        if ready is not None:      # lets the optimizer start this parameter's bucket reduction (parallel/ddp.py)
            ready()
        return None
    return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=w.dtype)


def _bias_grad(dy, b):
    if b is None:
        return None
    return colsum(dy, out_dtype=torch.float32).to(b.dtype)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        need_pre = act is not None and any(ctx.needs_input_grad[:3])
        if need_pre:
            y, pre = gemm(x, w, bias=b, epi=_ACT[act], want_aux=True)
        else:
            y, pre = gemm(x, w, bias=b, epi=_ACT[act]), None
        ctx.save_for_backward(x, w, pre)
        ctx.act = act
        ctx.has_bias = b is not None
        ctx.bias_ref = b
        ctx.w_param = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, pre = ctx.saved_tensors
        if dy.stride(1) != 1:
            dy = dy.contiguous()
        if ctx.act is not None:
            dy = act_bwd(dy, pre, ctx.act)
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dy, x, w, ctx.w_param) if ctx.needs_input_grad[1] else None
        db = _bias_grad(dy, ctx.bias_ref) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None


def linear(x, w, b=None, act=None):
    """act(x @ w.T + b) for 2-D bf16 x [rows, K] and w [N, K]."""
    if not x.is_cuda:
        y = F.linear(x, w, b)
        if act == "gelu":
            y = F.gelu(y, approximate="tanh")
        elif act == "silu":
            y = F.silu(y)
        return y
    return _Linear.apply(x, w, b, act)


class _LinearResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, res, gate, rows_per_gate):
        rows = x.shape[0]
        has_gate = gate is not None
        if has_gate:
            g = gate
            rpg = rows_per_gate
        else:
            g = torch.ones((1, w.shape[0]), dtype=torch.float32, device=x.device)
            rpg = rows
        need_z = has_gate and ctx.needs_input_grad[4]
        if need_z:
            y, z = gemm(x, w, bias=b, epi=EPI_GATE_RES, residual=res, gate=g, rows_per_gate=rpg, want_aux=True)
        else:
            y, z = gemm(x, w, bias=b, epi=EPI_GATE_RES, residual=res, gate=g, rows_per_gate=rpg), None
        ctx.save_for_backward(x, w, z, gate if has_gate else None)
        ctx.meta = (rows_per_gate, has_gate, b)
        ctx.w_param = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, z, gate = ctx.saved_tensors
        rows_per_gate, has_gate, b = ctx.meta
        if dy.stride(1) != 1:
            dy = dy.contiguous()
        rows, N = dy.shape
        dgate = None
        if has_gate:
            batch = (rows + rows_per_gate - 1) // rows_per_gate
            assert rows == batch * rows_per_gate
            dz = torch.empty((rows, N), dtype=torch.bfloat16, device=dy.device)
            want_dgate = ctx.needs_input_grad[4] and z is not None
            chunks = max(1, min(rows_per_gate, 592 // batch))
            partial = torch.empty((batch, chunks, N), dtype=torch.float32, device=dy.device)
            dgate = torch.empty((batch, N), dtype=torch.float32, device=dy.device) if want_dgate else None
            zz = z if z is not None else dy
            rc = _lib.lib().tt_gate_bwd(
                _lib.ptr(dy), _lib.c_ll(dy.stride(0)), _lib.ptr(zz), _lib.c_ll(zz.stride(0)), _lib.ptr(gate),
                _lib.c_ll(gate.stride(0)), _lib.ptr(dz), _lib.c_ll(N), _lib.ptr(partial), _lib.c_int(chunks),
                _lib.ptr(dgate), _lib.c_int(0), _lib.c_int(batch), _lib.c_int(rows_per_gate), _lib.c_int(N),
                _lib.stream())
            _lib.check(rc, "tt_gate_bwd")
        else:
            dz = dy
        dx = gemm(dz, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dz, x, w, ctx.w_param) if ctx.needs_input_grad[1] else None
        db = _bias_grad(dz, b) if (b is not None and ctx.needs_input_grad[2]) else None
        dres = dy if ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, dgate, None


def linear_residual(x, w, b, res, gate=None, rows_per_gate=1):
    """res + gate * (x @ w.T + b); gate fp32 [batch, N] (None = plain residual add)."""
    if not x.is_cuda:
        z = F.linear(x, w, b)
        if gate is not None:
            g = gate.float().repeat_interleave(rows_per_gate, dim=0)[: z.shape[0]]
            return (res.float() + g * z.float()).to(x.dtype)
        return res + z
    return _LinearResidual.apply(x, w, b, res, gate, rows_per_gate)


def ffn(x, w1, b1, w2, b2, res, gate=None, rows_per_gate=1, act="gelu"):
    """res + gate * (act(x @ w1.T + b1) @ w2.T + b2): the feed-forward branch of a DiT block
    (teletron/models/wan/wan_model.py:219-223, 264-265 in the reference)."""
    return linear_residual(linear(x, w1, b1, act), w2, b2, res, gate, rows_per_gate)
