"""Fused optimizer kernels over flat buffers (csrc/elementwise.cu): AdamW with fp32 master
weights and bf16 write-back, and the gradient L2 norm / clip coefficient.

Stand in for apex FusedAdam and amp_C.multi_tensor_l2norm used by the reference
(teletron/train/lr_scheduler.py:16,373-379, teletron/train/utils.py:262-268).
"""
from __future__ import annotations

import math

import torch

from . import _lib


def adamw_ref(p32, p16, m, v, g, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    """In-place fp32 reference of one AdamW step (decoupled weight decay)."""
    gg = g.float() * grad_scale
    m.mul_(beta1).add_(gg, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gg, gg, value=1 - beta2)
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    p32.sub_(lr * (mh / (vh.sqrt() + eps) + wd * p32))
    if p16 is not None:
        p16.copy_(p32.to(p16.dtype))


def adamw_step(p32, p16, m, v, g, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1,
               grad_scale=1.0, grad_scale_tensor=None, found_inf=None):
    """One AdamW step on flat fp32 buffers (element count a multiple of 4); p16 is the bf16 model copy."""
    if not p32.is_cuda:
        gs = grad_scale * (float(grad_scale_tensor) if grad_scale_tensor is not None else 1.0)
        if found_inf is not None and int(found_inf) != 0:
            return
        adamw_ref(p32, p16, m, v, g, lr, beta1, beta2, eps, wd, step, gs)
        return
    n = p32.numel()
    assert n % 4 == 0 and g.dtype == torch.float32 and g.numel() == n
    rc = _lib.lib().tt_adamw(
        _lib.ptr(p32), _lib.ptr(p16), _lib.ptr(m), _lib.ptr(v), _lib.ptr(g), _lib.c_ll(n), _lib.c_float(lr),
        _lib.c_float(beta1), _lib.c_float(beta2), _lib.c_float(eps), _lib.c_float(wd), _lib.c_int(step),
        _lib.ptr(grad_scale_tensor), _lib.c_float(grad_scale), _lib.ptr(found_inf), _lib.stream())
    _lib.check(rc, "tt_adamw")


def grad_norm(flat_grad: torch.Tensor, max_norm: float = 0.0) -> torch.Tensor:
    """Returns fp32[3] = (l2 norm, clip coefficient min(1, max_norm/(norm+1e-6)) or 1, sum of squares)."""
    if not flat_grad.is_cuda:
        ss = flat_grad.float().pow(2).sum()
        nrm = ss.sqrt()
        coef = torch.clamp(max_norm / (nrm + 1e-6), max=1.0) if max_norm > 0 else torch.ones(())
        return torch.stack([nrm, coef.to(nrm.dtype), ss])
    L = _lib.lib()
    n = flat_grad.numel()
    assert n % 4 == 0 and flat_grad.dtype == torch.float32
    partial = torch.empty(L.tt_sumsq_blocks(), dtype=torch.float32, device=flat_grad.device)
    out = torch.empty(3, dtype=torch.float32, device=flat_grad.device)
    rc = L.tt_grad_norm(_lib.ptr(flat_grad), _lib.c_ll(n), _lib.ptr(partial), _lib.c_float(max_norm),
                        _lib.ptr(out), _lib.stream())
    _lib.check(rc, "tt_grad_norm")
    return out
