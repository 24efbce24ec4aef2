"""Flow-matching elementwise ops (csrc/elementwise.cu): noising and the fused MSE loss.

``add_noise``   x_t = (1 - sigma) x0 + sigma * noise            (teletron/models/flow_match.py:62-68)
``flow_mse``    mean_b,n( w_b * (pred - (noise - x0))^2 ) with its gradient produced in the
                same pass                                         (examples/wan/pretrain_wan.py:58-61)
"""
from __future__ import annotations

import torch

from . import _lib


def add_noise_ref(x0, noise, sigma):
    s = sigma.float().view(-1, *([1] * (x0.dim() - 1)))
    return ((1.0 - s) * x0.float() + s * noise.float()).to(x0.dtype)


def add_noise(x0, noise, sigma):
    """x0, noise: [B, ...] bf16 contiguous; sigma: fp32 [B]."""
    if not x0.is_cuda or x0.dtype != torch.bfloat16 or (x0[0].numel() % 8) != 0:
        return add_noise_ref(x0, noise, sigma)
    x0c, nc = x0.contiguous(), noise.contiguous()
    out = torch.empty_like(x0c)
    sig = sigma.to(device=x0.device, dtype=torch.float32).contiguous()
    rc = _lib.lib().tt_add_noise(_lib.ptr(x0c), _lib.ptr(nc), _lib.ptr(out), _lib.c_ll(x0c[0].numel()),
                                 _lib.c_int(x0c.shape[0]), _lib.ptr(sig), _lib.stream())
    _lib.check(rc, "tt_add_noise")
    return out


def flow_mse_ref(pred, x0, noise, weight=None, denom=None):
    d = pred.float() - (noise.float() - x0.float())
    per = d.pow(2)
    if weight is not None:
        per = per * weight.float().view(-1, *([1] * (pred.dim() - 1)))
    n = denom if denom is not None else per.numel()
    return per.sum() / n


class _FlowMSE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pred, x0, noise, weight, scale):
        B = pred.shape[0]
        n = pred[0].numel()
        predc, x0c, nc = pred.contiguous(), x0.contiguous(), noise.contiguous()
        L = _lib.lib()
        blocks = L.tt_sumsq_blocks()
        partial = torch.empty(blocks, dtype=torch.float32, device=pred.device)
        loss = torch.empty((), dtype=torch.float32, device=pred.device)
        dpred = torch.empty_like(predc) if ctx.needs_input_grad[0] else None
        w = weight.to(device=pred.device, dtype=torch.float32).contiguous() if weight is not None else None
        rc = L.tt_flow_mse(_lib.ptr(predc), _lib.ptr(x0c), _lib.ptr(nc), _lib.ptr(dpred), _lib.c_ll(n),
                           _lib.c_int(B), _lib.ptr(w), _lib.c_float(scale), _lib.ptr(partial), _lib.ptr(loss),
                           _lib.stream())
        _lib.check(rc, "tt_flow_mse")
        ctx.save_for_backward(dpred)
        return loss * scale

    @staticmethod
    def backward(ctx, g):
        (dpred,) = ctx.saved_tensors
        # dpred already holds d(scale * loss)/dpred; g is 1 for a plain .backward()
        return dpred * g.to(dpred.dtype), None, None, None, None


def flow_mse(pred, x0, noise, weight=None, scale=1.0):
    """scale * mean(weight_b * (pred - (noise - x0))^2) over every element; differentiable in pred.

    ``scale`` lets a context-parallel rank that holds 1/P of the tokens contribute its share
    of the full-sequence mean (scale = 1/P), or fold 1/num_microbatches.
    """
    if not pred.is_cuda or pred.dtype != torch.bfloat16 or (pred[0].numel() % 8) != 0:
        return flow_mse_ref(pred, x0, noise, weight) * scale
    return _FlowMSE.apply(pred, x0, noise, weight, float(scale))
