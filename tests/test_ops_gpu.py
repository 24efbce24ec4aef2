"""Numerics of every CUDA kernel against its plain PyTorch fp32 reference (needs a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from teletron_b200 import ops
from teletron_b200.ops import _lib
import importlib

G = importlib.import_module("teletron_b200.ops.gemm")
N = importlib.import_module("teletron_b200.ops.norm")
from teletron_b200.ops.attention import attention_bwd, attention_fwd, attention_ref

DEV = "cuda"


def rel(a, b):
    a, b = a.float(), b.float()
    return (0.5 * (a - b).norm() / (a.norm() + b.norm() + 1e-30)).item()


@pytest.fixture(autouse=True)
def _seed_and_status():
    torch.manual_seed(0)
    yield
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N_,K", [(256, 256, 128), (1000, 1536, 328), (136, 72, 1000)])
def test_gemm_layouts(a_mn, b_mn, M, N_, K):
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N_) if b_mn else (N_, K), device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N_, device=DEV, dtype=torch.bfloat16)
    kw = dict(a_mn=bool(a_mn), b_mn=bool(b_mn), bias=bias, alpha=1.0 / math.sqrt(K))
    assert rel(G.gemm(a, b, **kw), G.gemm_ref(a, b, **kw)) < 2e-3


@pytest.mark.parametrize("epi", [G.EPI_GELU, G.EPI_SILU, G.EPI_GATE_RES, G.EPI_ACCUM])
def test_gemm_epilogues(epi):
    M, N_, K = 520, 384, 256
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N_, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N_, device=DEV, dtype=torch.bfloat16)
    kw = dict(bias=bias, epi=epi, alpha=1.0 / math.sqrt(K))
    if epi == G.EPI_GATE_RES:
        kw.update(residual=torch.randn(M, N_, device=DEV, dtype=torch.bfloat16),
                  gate=torch.randn(2, N_, device=DEV), rows_per_gate=260)
    if epi == G.EPI_ACCUM:
        base = torch.randn(M, N_, device=DEV, dtype=torch.float32)
        got = G.gemm(a, b, out=base.clone(), **kw)
        ref = G.gemm_ref(a, b, out=base.clone(), **kw)
        assert rel(got, ref) < 1e-4
        return
    got, aux = G.gemm(a, b, want_aux=True, **kw)
    ref, aux_ref = G.gemm_ref(a, b, want_aux=True, **kw)
    assert rel(got, ref) < 3e-3
    assert rel(aux, aux_ref) < 3e-3


@pytest.mark.parametrize("C", [256, 1536, 3072, 5120])
def test_adaln_fwd_bwd(C):
    B, S = 2, 77
    x = torch.randn(B * S, C, device=DEV).to(torch.bfloat16).requires_grad_(True)
    mod = (0.3 * torch.randn(B, 6, C, device=DEV)).requires_grad_(True)
    scale, shift = mod[:, 1], mod[:, 0]
    y = N.adaln(x, scale, shift, S)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    modr = mod.detach().clone().requires_grad_(True)
    yr = N.adaln_ref(xr, modr[:, 1], modr[:, 0], S)
    yr.backward(dy.float())
    assert rel(y, yr) < 3e-3
    assert rel(x.grad, xr.grad) < 5e-3
    assert rel(mod.grad, modr.grad) < 5e-3


def test_layernorm_affine():
    rows, C = 300, 1536
    x = torch.randn(rows, C, device=DEV).to(torch.bfloat16).requires_grad_(True)
    w = torch.randn(C, device=DEV).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(C, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = N.layernorm_affine(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (C,), wr, br, 1e-6)
    yr.backward(dy.float())
    assert rel(y, yr) < 3e-3 and rel(x.grad, xr.grad) < 5e-3
    assert rel(w.grad, wr.grad) < 1e-2 and rel(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("per_head,C", [(False, 1536), (True, 3072), (False, 5120)])
@pytest.mark.parametrize("with_rope", [True, False])
def test_rmsnorm_rope(per_head, C, with_rope):
    D, S, B = 128, 50, 2
    qkv = torch.randn(B * S, 3 * C, device=DEV).to(torch.bfloat16)
    x = qkv[:, C:2 * C].detach().requires_grad_(True)  # strided view, like a fused projection slice
    w = (1 + 0.1 * torch.randn(D if per_head else C, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    ang = torch.rand(S, D // 2, device=DEV) * 6.28
    freqs = torch.stack([ang.cos(), ang.sin()], -1).contiguous() if with_rope else None
    y = N.rmsnorm_rope(x, w, freqs, D, per_head)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = N.rmsnorm_rope_ref(xr, wr, freqs, D, per_head)
    yr.backward(dy.float())
    assert rel(y, yr) < 3e-3
    assert rel(x.grad, xr.grad) < 5e-3
    assert rel(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("B,Sq,Skv,H,kvl", [(1, 256, 256, 1, None), (2, 300, 1000, 3, None),
                                            (1, 1000, 520, 2, None), (2, 384, 512, 2, [257, 512]),
                                            (1, 64, 77, 1, None)])
def test_attention_fwd_bwd(B, Sq, Skv, H, kvl):
    D = 128
    q = torch.randn(B, Sq, H, D, device=DEV).to(torch.bfloat16)
    k = torch.randn(B, Skv, H, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(B, Skv, H, D, device=DEV).to(torch.bfloat16)
    do = torch.randn(B, Sq, H, D, device=DEV).to(torch.bfloat16)
    kv_lens = torch.tensor(kvl, dtype=torch.int32, device=DEV) if kvl else None
    o, lse = attention_fwd(q, k, v, kv_lens=kv_lens)
    dq, dk, dv = attention_bwd(q, k, v, o, lse, do, kv_lens=kv_lens)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    oref, lref = attention_ref(qf, kf, vf, kv_lens=kv_lens)
    oref.backward(do.float())
    assert rel(o, oref) < 2e-3 and (lse - lref).abs().max().item() < 1e-3
    assert rel(dq, qf.grad) < 3e-3 and rel(dk, kf.grad) < 3e-3 and rel(dv, vf.grad) < 3e-3


def test_attention_is_deterministic():
    q, k, v = (torch.randn(1, 512, 2, 128, device=DEV).to(torch.bfloat16) for _ in range(3))
    o1, l1 = attention_fwd(q, k, v)
    o2, l2 = attention_fwd(q, k, v)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    do = torch.randn_like(o1)
    g1 = attention_bwd(q, k, v, o1, l1, do)
    g2 = attention_bwd(q, k, v, o1, l1, do)
    assert all(torch.equal(a, b) for a, b in zip(g1, g2))


@pytest.mark.parametrize("act", [None, "gelu", "silu"])
def test_linear_autograd(act):
    rows, K, N_ = 333, 256, 384
    x = (torch.randn(rows, K, device=DEV) / 4).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N_, K, device=DEV) / 16).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(N_, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = ops.linear(x, w, b, act)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    if act == "gelu":
        yr = torch.nn.functional.gelu(yr, approximate="tanh")
    elif act == "silu":
        yr = torch.nn.functional.silu(yr)
    yr.backward(dy.float())
    assert rel(y, yr) < 3e-3 and rel(x.grad, xr.grad) < 5e-3
    assert rel(w.grad, wr.grad) < 5e-3 and rel(b.grad, br.grad) < 5e-3


def test_linear_residual_gate_and_main_grad():
    B, S, K, N_ = 2, 100, 256, 384
    rows = B * S
    x = (torch.randn(rows, K, device=DEV) / 4).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N_, K, device=DEV) / 16).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(N_, device=DEV).to(torch.bfloat16).requires_grad_(True)
    res = torch.randn(rows, N_, device=DEV).to(torch.bfloat16).requires_grad_(True)
    gate = torch.randn(B, N_, device=DEV).requires_grad_(True)
    w.main_grad = torch.full((N_, K), 0.5, device=DEV)
    y = ops.linear_residual(x, w, b, res, gate, S)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br, rr, gr = (t.detach().float().requires_grad_(True) for t in (x, w, b, res, gate))
    z = torch.nn.functional.linear(xr, wr, br)
    yr = rr + gr.repeat_interleave(S, 0) * z
    yr.backward(dy.float())
    assert rel(y, yr) < 3e-3 and rel(x.grad, xr.grad) < 6e-3 and rel(res.grad, rr.grad) < 1e-6
    assert rel(gate.grad, gr.grad) < 6e-3 and rel(b.grad, br.grad) < 6e-3
    assert w.grad is None and rel(w.main_grad - 0.5, wr.grad) < 6e-3


def test_weight_gradient_reaches_main_grad_under_activation_checkpointing():
    """Inside a non-reentrant checkpoint the backward pass gets a detached alias of the weight from its saved
    tensors, without the parameter's attributes.  The weight gradient must still be accumulated (fp32) into the
    parameter's main_grad and report through grad_ready, not come back as a bf16 ``.grad``."""
    from torch.utils.checkpoint import checkpoint

    B, S, K, F_, N_ = 2, 100, 256, 512, 256
    rows = B * S
    mk = lambda *sh, s=1.0: (torch.randn(*sh, device=DEV) * s).to(torch.bfloat16)
    x = mk(rows, K, s=0.5).requires_grad_(True)
    w1, b1 = torch.nn.Parameter(mk(F_, K, s=0.06)), torch.nn.Parameter(mk(F_))
    w2, b2 = torch.nn.Parameter(mk(N_, F_, s=0.04)), torch.nn.Parameter(mk(N_))
    res = mk(rows, N_)
    gate = torch.randn(B, N_, device=DEV)
    seen = []
    for name, w in (("w1", w1), ("w2", w2)):
        w.main_grad = torch.zeros(w.shape, device=DEV)
        w.grad_ready = (lambda n=name: seen.append(n))
    y = checkpoint(lambda t: ops.ffn(t, w1, b1, w2, b2, res, gate, S, act="gelu"), x, use_reentrant=False)
    dy = torch.randn_like(y)
    y.backward(dy)
    xx, a1, c1, a2, c2 = (t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2))
    h = torch.nn.functional.gelu(torch.nn.functional.linear(xx, a1, c1), approximate="tanh")
    yr = res.float() + gate.repeat_interleave(S, 0) * torch.nn.functional.linear(h, a2, c2)
    yr.backward(dy.float())
    assert w1.grad is None and w2.grad is None
    assert sorted(seen) == ["w1", "w2"]
    assert rel(w1.main_grad, a1.grad) < 8e-3 and rel(w2.main_grad, a2.grad) < 8e-3
    assert rel(x.grad, xx.grad) < 8e-3


@pytest.mark.parametrize("act", ["gelu", "silu"])
def test_ffn_matches_fp32_autograd(act):
    B, S, C, F_ = 2, 150, 256, 640
    rows = B * S
    mk = lambda *sh, s=1.0: (torch.randn(*sh, device=DEV) * s).to(torch.bfloat16)
    x, w1, b1, w2, b2, res = mk(rows, C, s=0.5), mk(F_, C, s=0.06), mk(F_), mk(C, F_, s=0.04), mk(C), mk(rows, C)
    gate = torch.randn(B, C, device=DEV)
    dy = torch.randn(rows, C, device=DEV).to(torch.bfloat16)
    ts = [t.detach().clone().requires_grad_(True) for t in (x, w1, b1, w2, b2, res, gate)]
    y1 = ops.ffn(*ts[:6], ts[6], S, act=act)
    y1.backward(dy)
    g1 = [t.grad for t in ts]
    ts = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2, res, gate)]
    xx, a1, c1, a2, c2, rr, gg = ts
    h = torch.nn.functional.linear(xx, a1, c1)
    h = torch.nn.functional.gelu(h, approximate="tanh") if act == "gelu" else torch.nn.functional.silu(h)
    yr = rr + gg.repeat_interleave(S, 0) * torch.nn.functional.linear(h, a2, c2)
    yr.backward(dy.float())
    assert rel(y1, yr) < 4e-3
    for name, u, v in zip("x w1 b1 w2 b2 res gate".split(), g1, [t.grad for t in ts]):
        assert rel(u, v) < 8e-3, (name, rel(u, v))


def test_flow_ops_and_adamw():
    B = 2
    x0, nz, pred = (torch.randn(B, 16, 3, 8, 8, device=DEV).to(torch.bfloat16) for _ in range(3))
    sig = torch.tensor([0.3, 0.9], device=DEV)
    assert rel(ops.add_noise(x0, nz, sig), ops.add_noise_ref(x0, nz, sig)) < 3e-3
    w = torch.tensor([0.7, 1.4], device=DEV)
    p = pred.clone().requires_grad_(True)
    loss = ops.flow_mse(p, x0, nz, w, scale=0.5)
    loss.backward()
    pr = pred.float().requires_grad_(True)
    lr_ = ops.flow_mse_ref(pr, x0, nz, w) * 0.5
    lr_.backward()
    assert abs(loss.item() - lr_.item()) < 1e-4 * abs(lr_.item()) + 1e-6
    assert rel(p.grad, pr.grad) < 5e-3
    n = 4096 + 64
    p32 = torch.randn(n, device=DEV); p16 = p32.to(torch.bfloat16)
    m = torch.zeros(n, device=DEV); v = torch.zeros(n, device=DEV); g = torch.randn(n, device=DEV)
    rp, rm, rv = p32.clone(), m.clone(), v.clone()
    for step in (1, 2, 3):
        ops.adamw_step(p32, p16, m, v, g, lr=1e-2, wd=0.1, step=step, grad_scale=0.5)
        ops.adamw_ref(rp, None, rm, rv, g, 1e-2, 0.9, 0.999, 1e-8, 0.1, step, 0.5)
    assert rel(p32, rp) < 1e-6 and rel(m, rm) < 1e-6 and rel(v, rv) < 1e-5
    assert torch.equal(p16, p32.to(torch.bfloat16))
    gn = ops.grad_norm(g, 1.0)
    assert abs(gn[0].item() - g.norm().item()) < 1e-3 * g.norm().item()


@pytest.mark.parametrize("world,seg,K,N,b_mn", [(2, 200, 192, 320, False), (3, 128, 256, 136, True), (2, 70, 64, 512, False)])
def test_gemm_ag_segments_on_one_device(world, seg, K, N, b_mn):
    """all-gather -> GEMM kernel with every "rank" buffer on this GPU (the kernel only sees device addresses)."""
    G = importlib.import_module("teletron_b200.ops.gemm")
    torch.manual_seed(0)
    segs = [torch.randn(seg, K, device="cuda").to(torch.bfloat16) for _ in range(world)]
    w = torch.randn(N, K, device="cuda").to(torch.bfloat16) * 0.1
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    b = w.t().contiguous() if b_mn else w
    y, pre = G.gemm_ag([t.data_ptr() for t in segs], seg, K, b, b_mn=b_mn, bias=bias, epi=G.EPI_GELU, want_aux=True)
    torch.cuda.synchronize()
    _lib.check_status()
    ref_pre = torch.cat(segs).float() @ w.float().t() + bias.float()
    ref = torch.nn.functional.gelu(ref_pre, approximate="tanh")
    assert rel(pre, ref_pre) < 4e-3
    assert rel(y, ref) < 4e-3


@pytest.mark.parametrize("world,seg,K,N,b_mn", [(2, 200, 192, 320, False), (3, 128, 256, 136, True),
                                                (2, 300, 128, 512, True), (4, 130, 320, 264, False)])
def test_gemm_rs_segments_on_one_device(world, seg, K, N, b_mn):
    """GEMM -> reduce-scatter: every emulated rank scatters its partial product into the owners' staging buffers,
    then each owner sums its slots."""
    G = importlib.import_module("teletron_b200.ops.gemm")
    torch.manual_seed(1)
    xs = [torch.randn(world * seg, K, device="cuda").to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(world)]
    staging = [torch.full((world, seg, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    ptrs = [t.data_ptr() for t in staging]
    for r in range(world):
        b = ws[r].t().contiguous() if b_mn else ws[r]
        G.gemm_rs_scatter(xs[r], b, ptrs, seg, r, b_mn=b_mn)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    total = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for s_ in range(world):
        out = G.tp_reduce_rows(staging[s_], world, seg, N, bias=bias)
        torch.cuda.synchronize()
        ref = total[s_ * seg:(s_ + 1) * seg] + bias.float()
        assert rel(out, ref) < 4e-3
    _lib.check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N_,K", [(520, 512, 192), (256, 776, 136), (1100, 264, 64)])
def test_gemm_pair_kernel_layouts(a_mn, b_mn, M, N_, K):
    """CTA-pair kernel (tcgen05.mma.cta_group::2) against the fp32 reference and the one-CTA kernel."""
    G = importlib.import_module("teletron_b200.ops.gemm")
    if a_mn:
        M = (M + 7) // 8 * 8
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N_) if b_mn else (N_, K), device="cuda").to(torch.bfloat16)
    old = G.set_pair_gemm(True)
    try:
        y2 = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        G.set_pair_gemm(False)
        y1 = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    finally:
        G.set_pair_gemm(old)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = G.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert rel(y2, ref) < 4e-3
    assert rel(y2, y1) < 1e-3


@pytest.mark.parametrize("epi", ["gelu", "gate_res", "accum_fp32", "bias"])
def test_gemm_pair_kernel_epilogues(epi):
    G = importlib.import_module("teletron_b200.ops.gemm")
    torch.manual_seed(1)
    M, N_, K = 700, 512, 256
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N_, K, device="cuda") * 0.1).to(torch.bfloat16)
    bias = torch.randn(N_, device="cuda").to(torch.bfloat16)
    kw = dict(bias=bias)
    if epi == "gelu":
        kw.update(epi=G.EPI_GELU, want_aux=True)
    elif epi == "gate_res":
        kw.update(epi=G.EPI_GATE_RES, residual=torch.randn(M, N_, device="cuda").to(torch.bfloat16),
                  gate=torch.randn(2, N_, device="cuda"), rows_per_gate=350, want_aux=True)
    elif epi == "accum_fp32":
        kw = dict(epi=G.EPI_ACCUM)
    outs = []
    for pair in (True, False):
        old = G.set_pair_gemm(pair)
        try:
            if epi == "accum_fp32":
                o = torch.full((M, N_), 0.5, device="cuda", dtype=torch.float32)
                G.gemm(a, b, out=o, **kw)
                outs.append((o,))
            else:
                r = G.gemm(a, b, **kw)
                outs.append(r if isinstance(r, tuple) else (r,))
        finally:
            G.set_pair_gemm(old)
    torch.cuda.synchronize()
    _lib.check_status()
    for x, y in zip(outs[0], outs[1]):
        assert rel(x, y) < 1e-3


# ------------------------------------------------------------------------------ real sizes, max-abs bounds, odd shapes
def _max_abs_ok(got, ref, frac):
    """Largest element-wise error relative to the reference's largest magnitude."""
    return (got.float() - ref.float()).abs().max().item() <= frac * ref.float().abs().max().item()


@pytest.mark.parametrize("M,N_,K,b_mn", [(2048, 1536, 8960, False), (1024, 5120, 13824, False), (2048, 8960, 1536, True)])
def test_gemm_at_the_models_reduction_depths(M, N_, K, b_mn):
    """K = 8,960 and 13,824 (the second feed-forward layer of the 1.3B / 14B models) accumulate 140 / 216 k-blocks
    per tile: normalised-L2 and max-abs error against the fp32 product."""
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N_) if b_mn else (N_, K), device=DEV, dtype=torch.bfloat16)
    kw = dict(b_mn=b_mn, alpha=1.0 / math.sqrt(K))
    ref = G.gemm_ref(a, b, out_dtype=torch.float32, **kw)
    for pair in (True, False):
        old = G.set_pair_gemm(pair)
        try:
            got = G.gemm(a, b, **kw)
        finally:
            G.set_pair_gemm(old)
        assert rel(got, ref) < 2e-3, (pair, rel(got, ref))
        assert _max_abs_ok(got, ref, 8e-3), pair      # bf16 output rounding of values up to ~5 sigma


def test_attention_at_the_benchmark_shape_rows_against_fp32():
    """32,760 tokens x 12 heads (the 480P x 81-frame sample): a few hundred query rows of the forward output, and
    dK / dV rows of the backward, against an fp32 softmax over all 32,760 keys."""
    S, H, D = 32760, 12, 128
    q, k, v = (torch.randn(1, S, H, D, device=DEV).to(torch.bfloat16) for _ in range(3))
    o, lse = attention_fwd(q, k, v)
    rows = torch.cat([torch.arange(0, 64), torch.arange(16300, 16364), torch.arange(S - 120, S)]).to(DEV)
    scale = 1.0 / math.sqrt(D)
    for h in (0, 7, 11):
        s = (q[0, rows, h].float() @ k[0, :, h].float().t()) * scale
        p = torch.softmax(s, dim=-1)
        ref = p @ v[0, :, h].float()
        got = o[0, rows, h]
        assert rel(got, ref) < 2e-3 and _max_abs_ok(got, ref, 2e-2), h
        assert (lse[0, h, rows] - torch.logsumexp(s, -1)).abs().max().item() < 2e-3
    # backward: dV = P^T dO and dK = dS^T Q for a slice of keys, with the probabilities of ALL queries of one head
    do = torch.randn_like(o)
    dq, dk, dv = attention_bwd(q, k, v, o, lse, do)
    h = 5
    keys = torch.arange(20000, 20128, device=DEV)
    s = (q[0, :, h].float() @ k[0, keys, h].float().t()) * scale                     # [S, 128]
    p = torch.exp(s - lse[0, h].unsqueeze(1))
    dv_ref = p.t() @ do[0, :, h].float()
    dp = do[0, :, h].float() @ v[0, keys, h].float().t()
    delta = (do[0, :, h].float() * o[0, :, h].float()).sum(-1, keepdim=True)
    dk_ref = (p * (dp - delta)).t() @ q[0, :, h].float() * scale
    assert rel(dv[0, keys, h], dv_ref) < 3e-3 and rel(dk[0, keys, h], dk_ref) < 5e-3
    assert _max_abs_ok(dv[0, keys, h], dv_ref, 3e-2) and _max_abs_ok(dk[0, keys, h], dk_ref, 3e-2)


@pytest.mark.parametrize("rows,C", [(65, 1536), (1, 256), (1027, 8960), (333, 72)])
def test_colsum_odd_shapes(rows, C):
    from teletron_b200.ops.linear import colsum

    x = torch.randn(rows, C, device=DEV).to(torch.bfloat16)
    ref = x.float().sum(0)
    got = colsum(x)
    assert (got - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    wide = torch.randn(rows, 2 * C + 8, device=DEV).to(torch.bfloat16)      # strided view
    assert (colsum(wide[:, 8:8 + C]) - wide[:, 8:8 + C].float().sum(0)).abs().max().item() <= \
        1e-4 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("n", [4, 1028, 999_996, 40_000_004])
def test_grad_norm_odd_lengths(n):
    from teletron_b200.ops.optim import grad_norm

    g = torch.randn(n, device=DEV)
    out = grad_norm(g, max_norm=1.0)
    ref = g.double().norm().item()
    assert abs(out[0].item() - ref) < 1e-5 * ref and abs(out[2].item() - ref * ref) < 1e-5 * ref * ref
    assert abs(out[1].item() - min(1.0, 1.0 / (ref + 1e-6))) < 1e-6


@pytest.mark.parametrize("B,S,C", [(1, 77, 1536), (2, 301, 256), (3, 64, 5120)])
def test_gate_backward_odd_shapes(B, S, C):
    """residual + gate * z: dz = gate * dy, dgate[b] = sum over the sample's rows of dy * z (two-stage column sums)."""
    rows = B * S
    mk = lambda *sh, s=1.0: (torch.randn(*sh, device=DEV) * s).to(torch.bfloat16)
    x, w, b, res = mk(rows, 128, s=0.5), mk(C, 128, s=0.1), mk(C), mk(rows, C)
    gate = torch.randn(B, C, device=DEV)
    dy = mk(rows, C)
    ts = [t.detach().clone().requires_grad_(True) for t in (x, w, b, res, gate)]
    ops.linear_residual(ts[0], ts[1], ts[2], ts[3], ts[4], S).backward(dy)
    rs = [t.detach().float().requires_grad_(True) for t in (x, w, b, res, gate)]
    z = torch.nn.functional.linear(rs[0], rs[1], rs[2])
    (rs[3] + rs[4].repeat_interleave(S, 0) * z).backward(dy.float())
    for name, u, v in zip("x w b res gate".split(), ts, rs):
        assert rel(u.grad, v.grad) < 8e-3, (name, rel(u.grad, v.grad))
    assert _max_abs_ok(ts[4].grad, rs[4].grad, 3e-2)


def test_multi_tensor_fold_matches_add():
    """Gradients of many small bf16 tensors folded into fp32 slices of a flat buffer in one launch per 48 tensors."""
    from teletron_b200.parallel.ddp import ParamBuffer

    torch.manual_seed(1)
    sizes = [7, 1536, 3, 9216, 128, 1] * 20                      # 120 tensors, odd lengths
    mod = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(n, device=DEV).to(torch.bfloat16)) for n in sizes])
    buf = ParamBuffer(mod)
    buf.grads.normal_()
    before = buf.grads.clone()
    for p in mod:
        p.grad = torch.randn_like(p)
    grads = {n: p.grad.clone() for n, p in buf.named}
    count0 = _lib.launch_count()
    buf.collect_grads()
    assert _lib.launch_count() - count0 == 3                      # ceil(120 / 48) launches
    for n, p in buf.named:
        o, cnt, _ = buf.index[n]
        assert torch.equal(buf.grads[o:o + cnt], before[o:o + cnt] + grads[n].float()), n
        assert p.grad is None


def test_tensor_map_cache_reuses_descriptors():
    L = _lib.lib()
    L.tt_tmap_cache_size.restype = _lib.c_ll
    a = torch.randn(512, 256, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(512, 256, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(512, 512, device=DEV, dtype=torch.bfloat16)
    G.gemm(a, b, out=out)
    n1 = L.tt_tmap_cache_size()
    for _ in range(5):
        G.gemm(a, b, out=out)
    assert L.tt_tmap_cache_size() == n1 and n1 >= 2
    assert rel(out, G.gemm_ref(a, b)) < 2e-3
