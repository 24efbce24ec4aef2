"""Ulysses attention with the all-to-alls fused into kernel epilogues over NVLink peer memory.

Per self-attention layer, forward:
  the q/k/v projection GEMM stores V straight into the owning peers' head-parallel buffers from its epilogue
  and leaves q, k (pre-norm) with their per-row sums of squares; the q/k RMSNorm+RoPE kernel takes the row
  statistics from there and stores its results into the owning peers' head-parallel buffers (seq -> head
  exchange as store patterns, no copy kernel)                              -> device barrier
  flash attention over [B, S, H/P, D]; its epilogue stores O both locally (kept for backward)
  and into the owning peer's sequence-parallel buffer (head -> seq exchange)  -> device barrier
backward mirrors it: dO is scattered to the head owners, the attention-backward kernels store
dQ / dK / dV into the token owners' staging buffers, and the RMSNorm+RoPE backward consumes them.

This replaces four NCCL all-to-alls per direction with no separate communication kernels and no
pack / unpack copies (reference: teletron/core/context_parallel/context_parallel_mixin.py:87-125).
Activations that must live until backward (q/k/v in head layout, O in sequence layout) are
taken from one symmetric slab used as a stack: a layer's region is released by its backward
(layers run backward in reverse order), at once when the forward pass is one whose activations
are dropped (the first pass of a checkpointed range, or no-grad evaluation), and the whole slab is
reset every micro-batch; gradient staging buffers are reused across layers.  Ordering across ranks
relies on every rank executing the same kernel sequence; each exchange is fenced by the bounded flag
barrier of csrc/comm.cu.
Requirements: head_dim 128, bf16, one NVLink box.  The head count need not divide by the group size: every rank
has ceil(H / P) head slots, the last ranks own fewer heads (or none) and run attention only over the heads they own.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import _lib
from ..ops.norm import rmsrope_bwd_raw
from ..utils.nvtx import nvtx_range
from .recompute import forward_is_discarded

_ALIGN = 128  # elements (256 bytes)


class SymmSlab:
    """Bump allocator over one symmetric bf16 buffer; identical call sequences on every rank give
    identical offsets, so peer addresses are base + offset."""

    def __init__(self, arena, numel: int):
        self.arena = arena
        self.buf = arena.alloc(numel, torch.bfloat16)
        self.numel = numel
        self.off = 0
        self.live = []
        self.high_water = 0

    def reset(self):
        self.off = 0
        self.live = []  # (start, end) of the regions that wait for their backward, in forward order

    def release_to(self, mark: int):
        self.off = mark

    def take(self, numel: int):
        n = (numel + _ALIGN - 1) // _ALIGN * _ALIGN
        if self.off + n > self.numel:
            raise RuntimeError(
                f"symmetric activation slab exhausted ({self.off + n} > {self.numel} elements); raise "
                "slab_bytes (FusedUlysses) or enable activation recompute")
        t = self.buf.tensor[self.off:self.off + numel]
        ptrs = self.buf.c_ptrs(self.off)
        self.off += n
        self.high_water = max(self.high_water, self.off)
        return t, ptrs


class FusedUlysses:
    def __init__(self, arena, slab_bytes: int = 0, barrier_slot: int = 2):
        self.arena = arena
        self.rank, self.world = arena.rank, arena.world
        self.slot = barrier_slot
        self.slab = SymmSlab(arena, slab_bytes // 2) if slab_bytes else None
        self._staging = {}
        # debugging aid (--poison-comm-buffers): before every micro-batch the slab and the gradient staging buffers are
        # filled with NaN, so a kernel that reads a peer's data before it has arrived produces NaN instead of stale,
        # plausible values (the race check that compute-sanitizer would otherwise do)
        self.poison = False
        self.seq_len: Optional[int] = None  # true (un-padded) global sequence length

    def supports(self, H: int, D: int) -> bool:
        return D == 128 and H >= 1

    def head_slots(self, H: int):
        """(slots per rank, heads this rank owns) for H heads over the group."""
        hl = (H + self.world - 1) // self.world
        return hl, max(0, min(hl, H - self.rank * hl))

    def begin_microbatch(self, need_elems: int = 0):
        """Call before the first layer of every forward pass: makes sure no peer still reads the slab
        regions of the previous micro-batch, then recycles the slab (growing it when ``need_elems``
        bf16 elements do not fit; every rank of the group takes the same decision)."""
        self.arena.barrier(self.slot)
        if self.slab is None or self.slab.numel < need_elems:
            torch.cuda.synchronize()
            self.slab = None
            self.slab = SymmSlab(self.arena, int(need_elems))
        self.slab.reset()
        if self.poison:
            with torch.autograd._unsafe_preserve_version_counter(self.slab.buf.tensor):
                self.slab.buf.tensor.fill_(float("nan"))
            for t in self._staging.values():
                t.tensor.fill_(float("nan"))
            self.arena.barrier(self.slot)      # nobody writes into a peer that is still poisoning

    @staticmethod
    def slab_elems(layers_alive: int, batch: int, s_pad: int, channels: int, world: int) -> int:
        """bf16 elements one micro-batch needs: per live layer q, k, v in head layout and O in sequence
        layout (4 tensors of about batch * s_pad * channels / world; head slots are rounded up when the head count
        does not divide by the group size), plus alignment slack."""
        heads = max(channels // 128, 1)
        slots = (heads + world - 1) // world
        per_layer = 3 * (batch * s_pad * slots * (channels // heads) + _ALIGN) + (batch * s_pad * channels // world + _ALIGN)
        return int(per_layer * max(layers_alive, 1) * 1.02) + 4 * _ALIGN

    def staging(self, name: str, numel: int):
        t = self._staging.get(name)
        if t is None or t.tensor.numel() < numel:
            t = self.arena.alloc(numel, torch.bfloat16)  # collective; same order on every rank
            self._staging[name] = t
        return t

    def attention_qkv(self, x, w_qkv, b_qkv, wq, wk, freqs, B, S_l, H, D, eps, scale=None):
        """Self-attention of x [B*S_l, K] from the fused projection weight w_qkv [3*H*D, K] on: projection (with
        the exchange of V in its epilogue), q/k norm + RoPE (exchange in its stores), attention (exchange of O
        in its epilogue).  Returns [B*S_l, H*D]."""
        # decided here: inside an autograd function's forward the grad mode is always off
        self._keep_for_backward = torch.is_grad_enabled() and not forward_is_discarded()
        return _FusedUlyssesFn.apply(self, x, w_qkv, b_qkv, wq, wk, freqs, B, S_l, H, D, eps, scale)

    def joint_attention(self, q_pre, k_pre, v, wq, wk, freqs, qt, kt, vt, text_lens, B, S_l, H, D, eps, scale=None):
        """Attention over [video tokens | replicated text tokens] (HunyuanVideo,
        teletron/models/hunyuan/parallel_model.py:84-118).  Video q_pre / k_pre / v: this rank's [B*S_l, H*D]
        projections before the per-head norm (wq / wk: [D]) and RoPE; they are normalised, rotated and stored into
        the head owners' joint buffers by the norm kernel.  Text qt / kt / vt: [B, T, H, D], already normalised and
        identical on every rank; each rank attends with its own heads of them.  text_lens [B] masks the padded
        text tail.  Returns (video output [B*S_l, H*D], this rank's heads of the text output [B, T, head slots, D]).
        The video token count must divide by the group size (no padding inside a joint sequence)."""
        self._keep_for_backward = torch.is_grad_enabled() and not forward_is_discarded()
        return _FusedJointFn.apply(self, q_pre, k_pre, v, wq, wk, freqs, qt, kt, vt, text_lens, B, S_l, H, D, eps,
                                   scale)


def _scatter_rows(fu: FusedUlysses, x, w, freqs, rstd, rows, C, D, eps, dst_ptrs, S_l, S_pad, ssq=None,
                  per_head=False, dst_rows=0):
    """norm (full row, or per head) + RoPE of x [rows, C] (either may be skipped: w / freqs None), stored with the
    seq -> head pattern into the peers' [B, dst_rows or S_pad, head slots, D] buffers."""
    L = _lib.lib()
    rc = L.tt_rmsrope_fwd_scatter(
        _lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(w), _lib.ptr(freqs),
        _lib.c_int(freqs.shape[0] if freqs is not None else 1), _lib.ptr(rstd), _lib.c_int(rows), _lib.c_int(C),
        _lib.c_int(D), _lib.c_int(int(per_head)), _lib.c_float(eps), dst_ptrs, _lib.c_int(fu.world),
        _lib.c_int(fu.rank), _lib.c_int(S_l), _lib.c_int(S_pad), _lib.ptr(ssq),
        _lib.c_int(ssq.shape[1] if ssq is not None else 0), _lib.c_ll(ssq.stride(0) if ssq is not None else 0),
        _lib.c_int(dst_rows), _lib.stream())
    _lib.check(rc, "tt_rmsrope_fwd_scatter")


class _FusedUlyssesFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fu: FusedUlysses, x, w_qkv, b_qkv, wq, wk, freqs, B, S_l, H, D, eps, scale):
        import math

        from ..ops.gemm import gemm

        P, rank = fu.world, fu.rank
        C = H * D
        Hl, heads = fu.head_slots(H)
        S_pad = S_l * P
        rows = B * S_l
        dev = x.device
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        n_h = B * S_pad * Hl * D
        slab_mark = fu.slab.off
        qh, qh_p = fu.slab.take(n_h)
        kh, kh_p = fu.slab.take(n_h)
        vh, vh_p = fu.slab.take(n_h)
        o_s, o_p = fu.slab.take(rows * C)
        wq_f = wq.float().contiguous()
        wk_f = wk.float().contiguous()
        rstd_q = torch.empty(rows, dtype=torch.float32, device=dev)
        rstd_k = torch.empty(rows, dtype=torch.float32, device=dev)
        L = _lib.lib()
        # K-QKV-A2A: projection GEMM whose epilogue stores V into the head owners and leaves the row statistics
        qk = torch.empty((rows, 2 * C), dtype=torch.bfloat16, device=dev)
        halves = C // 128
        ssq = torch.empty((rows, 2 * halves), dtype=torch.float32, device=dev) if C % 256 == 0 else None
        rc = -3
        if ssq is not None and x.stride(1) == 1 and w_qkv.stride(1) == 1:
            with nvtx_range("qkv_gemm_a2a"):
                rc = L.tt_gemm_qkv_a2a(
                    _lib.ptr(x), _lib.c_ll(x.stride(0)), _lib.ptr(w_qkv), _lib.c_ll(w_qkv.stride(0)),
                    _lib.ptr(b_qkv), _lib.ptr(qk), _lib.c_ll(qk.stride(0)), _lib.ptr(ssq), vh_p, _lib.c_int(P),
                    _lib.c_int(rank), _lib.c_int(rows), _lib.c_int(C), _lib.c_int(x.shape[1]), _lib.c_int(S_l),
                    _lib.c_int(H), _lib.c_int(D), _lib.ptr(_lib.status_word(dev)), _lib.stream())
        if rc == -3:      # too few rows for the CTA-pair kernel: plain GEMM, V exchanged by a copy kernel
            qkv = gemm(x, w_qkv, bias=b_qkv)
            qk, ssq = qkv, None
            _scatter_rows(fu, qkv[:, 2 * C:], None, None, None, rows, C, D, eps, vh_p, S_l, S_pad)
        else:
            _lib.check(rc, "tt_gemm_qkv_a2a")
        q_pre, k_pre = qk[:, 0:C], qk[:, C:2 * C]
        _scatter_rows(fu, q_pre, wq_f, freqs, rstd_q, rows, C, D, eps, qh_p, S_l, S_pad,
                      ssq[:, :halves] if ssq is not None else None)
        _scatter_rows(fu, k_pre, wk_f, freqs, rstd_k, rows, C, D, eps, kh_p, S_l, S_pad,
                      ssq[:, halves:] if ssq is not None else None)
        fu.arena.barrier(fu.slot)
        kv_lens = None
        if fu.seq_len is not None and fu.seq_len != S_pad:
            kv_lens = torch.full((B,), fu.seq_len, dtype=torch.int32, device=dev)
        o_h = lse = None
        if heads > 0:
            o_h = torch.empty(n_h, dtype=torch.bfloat16, device=dev)
            lse = torch.empty((B, heads, S_pad), dtype=torch.float32, device=dev)
            ld, bs = Hl * D, S_pad * Hl * D
            with nvtx_range("attn_fwd_a2a"):
                rc = L.tt_attn_fwd_scatter(
                    _lib.ptr(qh), _lib.c_ll(ld), _lib.c_ll(bs), _lib.ptr(kh), _lib.c_ll(ld), _lib.c_ll(bs),
                    _lib.ptr(vh), _lib.c_ll(ld), _lib.c_ll(bs), _lib.ptr(o_h), _lib.c_ll(ld), _lib.c_ll(bs),
                    _lib.ptr(lse), _lib.ptr(kv_lens), _lib.c_int(B), _lib.c_int(Hl), _lib.c_int(heads),
                    _lib.c_int(H), _lib.c_int(S_pad), _lib.c_int(S_pad), _lib.c_int(D), _lib.c_float(scale), o_p,
                    _lib.c_int(P), _lib.c_int(rank), _lib.ptr(_lib.status_word(dev)), _lib.stream())
            _lib.check(rc, "tt_attn_fwd_scatter")
        fu.arena.barrier(fu.slot)
        if not fu._keep_for_backward:
            # nothing of this layer is read after its own consumers (already enqueued): the next layer may
            # take the same region; its writers run behind this layer's last barrier on every rank
            fu.slab.release_to(slab_mark)
        else:
            fu.slab.live.append((slab_mark, fu.slab.off))
        ctx.fu = fu
        ctx.meta = (B, S_l, H, D, scale, kv_lens)
        ctx.save_for_backward(x, w_qkv, q_pre, k_pre, wq_f, wk_f, freqs, rstd_q, rstd_k, qh, kh, vh, o_h, lse)
        ctx.w_dtypes = (wq.dtype, wk.dtype)
        ctx.w_param = w_qkv
        ctx.bias_ref = b_qkv
        return o_s.view(rows, C)

    @staticmethod
    def backward(ctx, do):
        from ..ops.gemm import gemm
        from ..ops.linear import _bias_grad, _weight_grad

        fu: FusedUlysses = ctx.fu
        x, w_qkv, q_pre, k_pre, wq_f, wk_f, freqs, rstd_q, rstd_k, qh, kh, vh, o_h, lse = ctx.saved_tensors
        B, S_l, H, D, scale, kv_lens = ctx.meta
        P, rank = fu.world, fu.rank
        C, S_pad, rows = H * D, S_l * P, B * S_l
        Hl, heads = fu.head_slots(H)
        dev = do.device
        if do.stride(1) != 1:
            do = do.contiguous()
        n_h = B * S_pad * Hl * D
        do_h = fu.staging("do_h", n_h)
        # dQ, dK, dV land side by side in one [rows, 3C] matrix: the projection's gradient GEMMs read it in place
        dqkv_s = fu.staging("dqkv_s", rows * 3 * C)
        _scatter_rows(fu, do, None, None, None, rows, C, D, 0.0, do_h.c_ptrs(), S_l, S_pad)
        fu.arena.barrier(fu.slot)
        L = _lib.lib()
        if heads > 0:
            L.tt_attn_bwd_scratch_floats.restype = _lib.c_ll
            scratch = torch.empty(L.tt_attn_bwd_scratch_floats(_lib.c_int(B), _lib.c_int(heads), _lib.c_int(S_pad)),
                                  dtype=torch.float32, device=dev)
            with nvtx_range("attn_bwd_a2a"):
                rc = L.tt_attn_bwd_scatter(
                    _lib.ptr(qh), _lib.ptr(kh), _lib.ptr(vh), _lib.ptr(o_h), _lib.ptr(do_h.tensor), _lib.ptr(lse),
                    _lib.ptr(scratch), dqkv_s.c_ptrs(0), dqkv_s.c_ptrs(C), dqkv_s.c_ptrs(2 * C), _lib.c_ll(3 * C),
                    None, None, None, _lib.ptr(kv_lens), _lib.c_int(B), _lib.c_int(Hl), _lib.c_int(heads),
                    _lib.c_int(H), _lib.c_int(S_pad), _lib.c_int(S_pad), _lib.c_int(D), _lib.c_float(scale),
                    _lib.c_int(P), _lib.c_int(rank), _lib.ptr(_lib.status_word(dev)), _lib.stream())
            _lib.check(rc, "tt_attn_bwd_scatter")
        fu.arena.barrier(fu.slot)
        dqkv = dqkv_s.tensor[:rows * 3 * C].view(rows, 3 * C)
        # norm + rope backward in place on the q and k column blocks (each thread rewrites only what it has read)
        _, dwq = rmsrope_bwd_raw(dqkv[:, 0:C], q_pre, wq_f, freqs, rstd_q, D, False, out=dqkv[:, 0:C])
        _, dwk = rmsrope_bwd_raw(dqkv[:, C:2 * C], k_pre, wk_f, freqs, rstd_k, D, False, out=dqkv[:, C:2 * C])
        dx = gemm(dqkv, w_qkv, b_mn=True) if ctx.needs_input_grad[1] else None
        dw = _weight_grad(dqkv, x, w_qkv, ctx.w_param) if ctx.needs_input_grad[2] else None
        db = _bias_grad(dqkv, ctx.bias_ref) if (ctx.bias_ref is not None and ctx.needs_input_grad[3]) else None
        # layers run backward in reverse order, so this layer's region is the top of the stack
        if fu.slab.live and fu.slab.live[-1][1] == fu.slab.off:
            fu.slab.release_to(fu.slab.live.pop()[0])
        wdq, wdk = ctx.w_dtypes
        return (None, dx, dw, db, dwq.to(wdq), dwk.to(wdk), None, None, None, None, None, None, None)


class _FusedJointFn(torch.autograd.Function):
    """Joint video + text attention with the video exchanges in the kernels' stores; the text tokens never leave
    the rank (every rank holds them and uses its own heads)."""

    @staticmethod
    def forward(ctx, fu: FusedUlysses, q_pre, k_pre, v, wq, wk, freqs, qt, kt, vt, text_lens, B, S_l, H, D, eps, scale):
        import math

        P, rank = fu.world, fu.rank
        C = H * D
        Hl, heads = fu.head_slots(H)
        assert heads == Hl, "joint attention needs the head count to divide by the group size"
        S_pad = S_l * P
        T = qt.shape[1]
        Tp = (T + 7) // 8 * 8
        S_tot = S_pad + Tp
        rows = B * S_l
        dev = q_pre.device
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        n_h = B * S_tot * Hl * D
        slab_mark = fu.slab.off
        qh, qh_p = fu.slab.take(n_h)
        kh, kh_p = fu.slab.take(n_h)
        vh, vh_p = fu.slab.take(n_h)
        o_s, o_p = fu.slab.take(rows * C)
        wq_f, wk_f = wq.float().contiguous(), wk.float().contiguous()
        rstd_q = torch.empty((rows, H), dtype=torch.float32, device=dev)
        rstd_k = torch.empty((rows, H), dtype=torch.float32, device=dev)
        with nvtx_range("joint_qkv_a2a"):
            _scatter_rows(fu, q_pre, wq_f, freqs, rstd_q, rows, C, D, eps, qh_p, S_l, S_pad, per_head=True, dst_rows=S_tot)
            _scatter_rows(fu, k_pre, wk_f, freqs, rstd_k, rows, C, D, eps, kh_p, S_l, S_pad, per_head=True, dst_rows=S_tot)
            _scatter_rows(fu, v, None, None, None, rows, C, D, eps, vh_p, S_l, S_pad, dst_rows=S_tot)
        # this rank's heads of the text tokens go behind the video rows of the same buffers (no concatenation)
        # (every slab view shares one version counter with the slab; these writes, like the kernels' own, must not
        # look to autograd like changes to the earlier layers' saved q / k / v)
        hs = slice(rank * Hl, (rank + 1) * Hl)
        with torch.autograd._unsafe_preserve_version_counter(fu.slab.buf.tensor):
            for buf, t in ((qh, qt), (kh, kt), (vh, vt)):
                b4 = buf.view(B, S_tot, Hl, D)
                b4[:, S_pad:S_pad + T].copy_(t[:, :, hs])
                if Tp > T:
                    b4[:, S_pad + T:].zero_()
        fu.arena.barrier(fu.slot)
        kv_lens = (text_lens.to(device=dev, dtype=torch.int32) + S_pad) if text_lens is not None else \
            torch.full((B,), S_pad + T, dtype=torch.int32, device=dev)
        o_h = torch.empty(n_h, dtype=torch.bfloat16, device=dev)
        lse = torch.empty((B, Hl, S_tot), dtype=torch.float32, device=dev)
        ld, bs = Hl * D, S_tot * Hl * D
        L = _lib.lib()
        with nvtx_range("joint_attn_fwd_a2a"):
            rc = L.tt_attn_fwd_scatter(
                _lib.ptr(qh), _lib.c_ll(ld), _lib.c_ll(bs), _lib.ptr(kh), _lib.c_ll(ld), _lib.c_ll(bs),
                _lib.ptr(vh), _lib.c_ll(ld), _lib.c_ll(bs), _lib.ptr(o_h), _lib.c_ll(ld), _lib.c_ll(bs),
                _lib.ptr(lse), _lib.ptr(kv_lens), _lib.c_int(B), _lib.c_int(Hl), _lib.c_int(Hl), _lib.c_int(H),
                _lib.c_int(S_pad), _lib.c_int(S_tot), _lib.c_int(D), _lib.c_float(scale), o_p, _lib.c_int(P),
                _lib.c_int(rank), _lib.ptr(_lib.status_word(dev)), _lib.stream())
        _lib.check(rc, "tt_attn_fwd_scatter")
        fu.arena.barrier(fu.slot)
        ot = o_h.view(B, S_tot, Hl, D)[:, S_pad:S_pad + T].clone()
        if not fu._keep_for_backward:
            fu.slab.release_to(slab_mark)
        else:
            fu.slab.live.append((slab_mark, fu.slab.off))
        ctx.fu = fu
        ctx.meta = (B, S_l, H, D, T, Tp, scale)
        ctx.save_for_backward(q_pre, k_pre, wq_f, wk_f, freqs, rstd_q, rstd_k, qh, kh, vh, o_h, lse, kv_lens)
        ctx.w_dtypes = (wq.dtype, wk.dtype)
        ctx.text_shape = tuple(qt.shape)
        return o_s.view(rows, C), ot

    @staticmethod
    def backward(ctx, do, dot):
        fu: FusedUlysses = ctx.fu
        q_pre, k_pre, wq_f, wk_f, freqs, rstd_q, rstd_k, qh, kh, vh, o_h, lse, kv_lens = ctx.saved_tensors
        B, S_l, H, D, T, Tp, scale = ctx.meta
        P, rank = fu.world, fu.rank
        C, S_pad, rows = H * D, S_l * P, B * S_l
        Hl = H // P
        S_tot = S_pad + Tp
        dev = do.device
        if do.stride(1) != 1:
            do = do.contiguous()
        n_h = B * S_tot * Hl * D
        do_h = fu.staging("do_h", n_h)
        dqkv_s = fu.staging("dqkv_s", rows * 3 * C)
        _scatter_rows(fu, do, None, None, None, rows, C, D, 0.0, do_h.c_ptrs(), S_l, S_pad, dst_rows=S_tot)
        d4 = do_h.tensor[:n_h].view(B, S_tot, Hl, D)
        d4[:, S_pad:S_pad + T].copy_(dot)
        if Tp > T:
            d4[:, S_pad + T:].zero_()
        fu.arena.barrier(fu.slot)
        L = _lib.lib()
        L.tt_attn_bwd_scratch_floats.restype = _lib.c_ll
        scratch = torch.empty(L.tt_attn_bwd_scratch_floats(_lib.c_int(B), _lib.c_int(Hl), _lib.c_int(S_tot)),
                              dtype=torch.float32, device=dev)
        # gradients of the rows that stay local (text): head-layout buffers of the joint length
        dql, dkl, dvl = (torch.empty(n_h, dtype=torch.bfloat16, device=dev) for _ in range(3))
        with nvtx_range("joint_attn_bwd_a2a"):
            rc = L.tt_attn_bwd_scatter(
                _lib.ptr(qh), _lib.ptr(kh), _lib.ptr(vh), _lib.ptr(o_h), _lib.ptr(do_h.tensor), _lib.ptr(lse),
                _lib.ptr(scratch), dqkv_s.c_ptrs(0), dqkv_s.c_ptrs(C), dqkv_s.c_ptrs(2 * C), _lib.c_ll(3 * C),
                _lib.ptr(dql), _lib.ptr(dkl), _lib.ptr(dvl), _lib.ptr(kv_lens), _lib.c_int(B), _lib.c_int(Hl),
                _lib.c_int(Hl), _lib.c_int(H), _lib.c_int(S_pad), _lib.c_int(S_tot), _lib.c_int(D),
                _lib.c_float(scale), _lib.c_int(P), _lib.c_int(rank), _lib.ptr(_lib.status_word(dev)), _lib.stream())
        _lib.check(rc, "tt_attn_bwd_scatter")
        fu.arena.barrier(fu.slot)
        dqkv = dqkv_s.tensor[:rows * 3 * C].view(rows, 3 * C)
        dq_pre, dwq = rmsrope_bwd_raw(dqkv[:, 0:C], q_pre, wq_f, freqs, rstd_q, D, True)
        dk_pre, dwk = rmsrope_bwd_raw(dqkv[:, C:2 * C], k_pre, wk_f, freqs, rstd_k, D, True)
        dv = dqkv[:, 2 * C:].clone()
        # text gradients: this rank's heads only, the other heads' slots are zero (their owners contribute them)
        hs = slice(rank * Hl, (rank + 1) * Hl)
        outs = []
        for g in (dql, dkl, dvl):
            full = torch.zeros(ctx.text_shape, dtype=torch.bfloat16, device=dev)
            full[:, :, hs] = g.view(B, S_tot, Hl, D)[:, S_pad:S_pad + T]
            outs.append(full)
        if fu.slab.live and fu.slab.live[-1][1] == fu.slab.off:
            fu.slab.release_to(fu.slab.live.pop()[0])
        wdq, wdk = ctx.w_dtypes
        return (None, dq_pre, dk_pre, dv, dwq.to(wdq), dwk.to(wdk), None, outs[0], outs[1], outs[2], None,
                None, None, None, None, None, None)
