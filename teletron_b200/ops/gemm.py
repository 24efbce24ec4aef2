"""bf16 GEMM on tcgen05 tensor cores (csrc/gemm.cu) and the autograd Linear built on it.

``gemm`` computes ``C[M,N] = epilogue(alpha * A @ B^T)`` where either operand may be
stored transposed ("MN-major"), so forward, dgrad and wgrad of a Linear layer need no
transpose pass.  ``gemm_ref`` is the fp32 PyTorch statement of the same contract and is
what runs on CPU.  Replaces cuBLAS behind ``nn.Linear`` in the reference
(teletron/models/wan/wan_model.py:144-147).
"""
from __future__ import annotations

import torch

from . import _lib

EPI_NONE, EPI_GELU, EPI_GATE_RES, EPI_ACCUM, EPI_SILU = 0, 1, 2, 3, 4

# CTA-pair kernel (csrc/gemm2.cu, tcgen05.mma.cta_group::2) for outputs of at least 256 x 256; the one-CTA kernel
# (csrc/gemm.cu) takes everything else.
_PAIR = True


def set_pair_gemm(on: bool) -> bool:
    """Route large GEMMs to the CTA-pair kernel (default) or everything to the one-CTA kernel, which the tests use
    to cover both; returns the previous setting."""
    global _PAIR
    old, _PAIR = _PAIR, bool(on)
    return old


def _logical(a: torch.Tensor, mn_major: bool) -> torch.Tensor:
    return a.t() if mn_major else a


def gemm_ref(a, b, *, a_mn=False, b_mn=False, bias=None, epi=EPI_NONE, residual=None, gate=None,
             rows_per_gate=1, out=None, out_dtype=torch.bfloat16, alpha=1.0, want_aux=False):
    """fp32 reference. A logical [M,K], B logical [N,K]."""
    A = _logical(a, a_mn).float()
    B = _logical(b, b_mn).float()
    acc = alpha * (A @ B.t())
    if bias is not None:
        acc = acc + bias.float()
    aux = None
    if epi == EPI_GELU:
        aux = acc.to(torch.bfloat16) if want_aux else None
        acc = torch.nn.functional.gelu(acc, approximate="tanh")
    elif epi == EPI_SILU:
        aux = acc.to(torch.bfloat16) if want_aux else None
        acc = torch.nn.functional.silu(acc)
    elif epi == EPI_GATE_RES:
        aux = acc.to(torch.bfloat16) if want_aux else None
        g = gate.float().repeat_interleave(rows_per_gate, dim=0)[: acc.shape[0]]
        acc = residual.float() + g * acc
    elif epi == EPI_ACCUM:
        acc = out.float() + acc
    if out is not None:
        out.copy_(acc.to(out.dtype))
        res = out
    else:
        res = acc.to(out_dtype)
    return (res, aux) if want_aux else res


def gemm(a, b, *, a_mn=False, b_mn=False, bias=None, epi=EPI_NONE, residual=None, gate=None,
         rows_per_gate=1, out=None, out_dtype=torch.bfloat16, alpha=1.0, want_aux=False, max_ctas=0, aux=None):
    """C = epilogue(alpha * A @ B^T).

    a: [M,K] (or [K,M] when a_mn)   b: [N,K] (or [K,N] when b_mn); both bf16 with a
    contiguous last dim.  ``epi``: EPI_GELU / EPI_SILU (optionally returning the
    pre-activation as aux), EPI_GATE_RES (``residual + gate[row // rows_per_gate] * acc``,
    gate fp32), EPI_ACCUM (``out += acc``).
    """
    if not a.is_cuda:
        return gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, epi=epi, residual=residual, gate=gate,
                        rows_per_gate=rows_per_gate, out=out, out_dtype=out_dtype, alpha=alpha,
                        want_aux=want_aux)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm operands must be bf16"
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
    if want_aux:
        if aux is None:
            aux = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        assert aux.shape == (M, N) and out.stride(0) == aux.stride(0)
    else:
        aux = None
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == N
    if epi == EPI_GATE_RES:
        assert residual.dtype == torch.bfloat16 and gate.dtype == torch.float32
        assert residual.shape == (M, N) and residual.stride(1) == 1 and gate.stride(-1) == 1
    L = _lib.lib()
    if _PAIR and max_ctas == 0 and M >= 256 and N >= 256:
        rc = L.tt_gemm2_bf16(
            _lib.ptr(a), _lib.c_ll(a.stride(0)), _lib.c_int(int(a_mn)),
            _lib.ptr(b), _lib.c_ll(b.stride(0)), _lib.c_int(int(b_mn)),
            _lib.ptr(out), _lib.c_ll(out.stride(0)), _lib.c_int(int(out.dtype == torch.float32)),
            _lib.c_int(M), _lib.c_int(N), _lib.c_int(K), _lib.ptr(bias), _lib.c_int(epi),
            _lib.ptr(residual), _lib.c_ll(residual.stride(0) if residual is not None else 0),
            _lib.ptr(gate), _lib.c_ll(gate.stride(0) if gate is not None else 0),
            _lib.c_int(rows_per_gate), _lib.ptr(aux), _lib.c_float(alpha),
            _lib.ptr(_lib.status_word(a.device)), _lib.stream())
        if rc != -3:
            _lib.check(rc, "tt_gemm2_bf16")
            return (out, aux) if want_aux else out
    rc = L.tt_gemm_bf16(
        _lib.ptr(a), _lib.c_ll(a.stride(0)), _lib.c_int(int(a_mn)),
        _lib.ptr(b), _lib.c_ll(b.stride(0)), _lib.c_int(int(b_mn)),
        _lib.ptr(out), _lib.c_ll(out.stride(0)), _lib.c_int(int(out.dtype == torch.float32)),
        _lib.c_int(M), _lib.c_int(N), _lib.c_int(K), _lib.ptr(bias), _lib.c_int(epi),
        _lib.ptr(residual), _lib.c_ll(residual.stride(0) if residual is not None else 0),
        _lib.ptr(gate), _lib.c_ll(gate.stride(0) if gate is not None else 0),
        _lib.c_int(rows_per_gate), _lib.ptr(aux), _lib.c_float(alpha),
        _lib.ptr(_lib.status_word(a.device)), _lib.c_int(max_ctas), _lib.stream())
    _lib.check(rc, "tt_gemm_bf16")
    return (out, aux) if want_aux else out


# ------------------------------------------------------------------------------ tensor-parallel variants
def gemm_ag(a_peer_ptrs, seg_rows: int, k: int, b, *, b_mn=False, bias=None, epi=EPI_NONE, want_aux=False,
            device=None):
    """all-gather -> GEMM in one kernel: ``C = epilogue([A_0; A_1; ...] @ B^T)`` where segment s of A
    ([seg_rows, k], row stride k) is read from rank s's buffer at device address ``a_peer_ptrs[s]``
    (csrc/gemm.cu, tt_gemm_bf16_ag).  The caller has put a barrier between the writes of A and this call."""
    world = len(a_peer_ptrs)
    n = b.shape[1] if b_mn else b.shape[0]
    assert b.dtype == torch.bfloat16 and b.stride(1) == 1
    out = torch.empty((world * seg_rows, n), dtype=torch.bfloat16, device=device or b.device)
    aux = torch.empty_like(out) if want_aux else None
    ptrs = (_lib.c_ll * world)(*[int(p) for p in a_peer_ptrs])
    rc = _lib.lib().tt_gemm_bf16_ag(ptrs, _lib.c_ll(k), _lib.ptr(b), _lib.c_ll(b.stride(0)), _lib.c_int(int(b_mn)),
                                    _lib.ptr(out), _lib.c_ll(out.stride(0)), _lib.c_int(seg_rows), _lib.c_int(world),
                                    _lib.c_int(n), _lib.c_int(k), _lib.ptr(bias), _lib.c_int(epi), _lib.ptr(aux),
                                    _lib.ptr(_lib.status_word(out.device)), _lib.stream())
    _lib.check(rc, "tt_gemm_bf16_ag")
    return (out, aux) if want_aux else out


def gemm_ag_gather(a_peer_ptrs, seg_rows: int, k: int, b, flags, epoch: int, rank: int, *, b_mn=False, bias=None,
                   epi=EPI_NONE, want_aux=False, device=None):
    """all-gather -> GEMM in one kernel that gathers as it multiplies (csrc/gemm2.cu, tt_gemm2_bf16_ag): segment s of
    A is read once from rank s's buffer by the kernel's copier warps into a local gathered matrix, which is returned
    as the third result.  ``flags``: int32 [>= ceil(world * seg_rows / 128)] holding no value equal to ``epoch``."""
    world = len(a_peer_ptrs)
    n = b.shape[1] if b_mn else b.shape[0]
    assert b.dtype == torch.bfloat16 and b.stride(1) == 1
    dev = device or b.device
    out = torch.empty((world * seg_rows, n), dtype=torch.bfloat16, device=dev)
    aux = torch.empty_like(out) if want_aux else None
    gathered = torch.empty((world * seg_rows, k), dtype=torch.bfloat16, device=dev)
    ptrs = (_lib.c_ll * world)(*[int(p) for p in a_peer_ptrs])
    rc = _lib.lib().tt_gemm2_bf16_ag(ptrs, _lib.ptr(b), _lib.c_ll(b.stride(0)), _lib.c_int(int(b_mn)), _lib.ptr(out),
                                     _lib.c_ll(out.stride(0)), _lib.ptr(gathered), _lib.ptr(flags), _lib.c_uint(epoch),
                                     _lib.c_int(seg_rows), _lib.c_int(world), _lib.c_int(rank), _lib.c_int(n),
                                     _lib.c_int(k), _lib.ptr(bias), _lib.c_int(epi), _lib.ptr(aux),
                                     _lib.ptr(_lib.status_word(dev)), _lib.stream())
    _lib.check(rc, "tt_gemm2_bf16_ag")
    return out, aux, gathered


def gemm_rs_scatter(a, b, c_peer_ptrs, seg_rows: int, rank: int, *, b_mn=False):
    """First half of GEMM -> reduce-scatter: the partial product ``a @ b^T`` ([world * seg_rows, n]) is stored,
    tile by tile, into slot ``rank`` of the staging buffer ([world, seg_rows, n]) of the rank that owns the rows
    (csrc/gemm2.cu, tt_gemm2_bf16_rs on CTA pairs; csrc/gemm.cu, tt_gemm_bf16_rs for small shapes)."""
    world = len(c_peer_ptrs)
    n = b.shape[1] if b_mn else b.shape[0]
    m, k = a.shape
    assert m == world * seg_rows and a.stride(1) == 1 and b.stride(1) == 1
    ptrs = (_lib.c_ll * world)(*[int(p) for p in c_peer_ptrs])
    if _PAIR:
        rc = _lib.lib().tt_gemm2_bf16_rs(_lib.ptr(a), _lib.c_ll(a.stride(0)), _lib.ptr(b), _lib.c_ll(b.stride(0)),
                                         _lib.c_int(int(b_mn)), ptrs, _lib.c_ll(n), _lib.c_int(seg_rows),
                                         _lib.c_int(world), _lib.c_int(rank), _lib.c_int(n), _lib.c_int(k),
                                         _lib.ptr(_lib.status_word(a.device)), _lib.stream())
        if rc != -3:
            _lib.check(rc, "tt_gemm2_bf16_rs")
            return
    rc = _lib.lib().tt_gemm_bf16_rs(_lib.ptr(a), _lib.c_ll(a.stride(0)), _lib.ptr(b), _lib.c_ll(b.stride(0)),
                                    _lib.c_int(int(b_mn)), ptrs, _lib.c_ll(n), _lib.c_int(seg_rows), _lib.c_int(world),
                                    _lib.c_int(rank), _lib.c_int(n), _lib.c_int(k),
                                    _lib.ptr(_lib.status_word(a.device)), _lib.stream())
    _lib.check(rc, "tt_gemm_bf16_rs")


def tp_reduce_rows(staging, world: int, rows: int, n: int, bias=None):
    """Second half: ``out[r] = bias + sum_w staging[w, r]`` (fp32 accumulation)."""
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=staging.device)
    rc = _lib.lib().tt_tp_reduce_rows(_lib.ptr(staging), _lib.c_int(world), _lib.c_ll(rows), _lib.c_int(n), _lib.c_ll(n),
                                      _lib.ptr(bias), _lib.ptr(out), _lib.c_ll(n), _lib.stream())
    _lib.check(rc, "tt_tp_reduce_rows")
    return out
