"""Small, self-contained workloads for profiling single kernels (``ncu -k regex:<kernel> -c 1 ...``).

    python examples/profiling/profile_cases.py gemm  [--m 32760 --n 8960 --k 1536 --epi gelu]
    python examples/profiling/profile_cases.py attn  [--seq 16384 --heads 12] [--bwd]
    python examples/profiling/profile_cases.py norm  [--rows 32760 --c 1536]
    python examples/profiling/profile_cases.py layers [--layers 2]     Wan2.1-1.3B blocks, one 480P x 81 sample, fwd + bwd

Each case runs one warm-up and then a few timed launches (CUDA events) and prints the achieved
rate, so the same command serves both as the plain run and as the profiled run.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from teletron_b200.ops import _lib  # noqa: E402
from teletron_b200.ops.attention import attention_bwd, attention_fwd  # noqa: E402
from teletron_b200.ops.gemm import EPI_GELU, EPI_NONE, gemm  # noqa: E402
from teletron_b200.ops.norm import adaln  # noqa: E402


def _time(fn, iters=3):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _tp_case(a):
    """Column-parallel + row-parallel linear pair (an MLP), forward + backward, under torchrun on the ranks of one box:
    ``--rows`` tokens per rank, hidden ``--c``, inner width ``--inner`` (sharded).  Max over ranks of the device time."""
    import os

    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.parallel.tp import ColumnParallelLinear, FusedTP, RowParallelLinear, TPContext

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    tp = TPContext(dist.group.WORLD, world, rank)
    if a.fused:
        tp.fused = FusedTP(SymmetricArena(dist.group.WORLD))
    torch.manual_seed(0)
    col = ColumnParallelLinear(a.c, a.inner, tp).cuda().to(torch.bfloat16)
    row = RowParallelLinear(a.inner, a.c, tp).cuda().to(torch.bfloat16)
    x = torch.randn(a.rows, a.c, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(a.rows, a.c, device="cuda", dtype=torch.bfloat16)

    def step():
        x.grad = None
        row(col(x, act="gelu")).backward(dy)

    for _ in range(3):
        step()
    dist.barrier()
    ms = _time(step, a.iters)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    _lib.check_status()
    if rank == 0:
        flops = 3 * 2 * 2.0 * a.rows * world * a.c * (a.inner / world)  # fwd + dgrad + wgrad of both linears, per rank
        print(json.dumps(dict(case="tp", world=world, fused=bool(a.fused), rows_per_rank=a.rows, c=a.c, inner=a.inner,
                              ms=float(t.item()), tflops_per_rank=flops / float(t.item()) / 1e9)), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def _dpopt_case(a):
    """Data-parallel gradient reduce-scatter + clip + AdamW + parameter all-gather of a flat buffer of ``--params``
    million bf16 parameters with fp32 gradients, under torchrun on the ranks of one box.  ``--fused``: the peer-memory
    kernels (pull-reduce of the owned shard from every peer, AdamW, parameter store into every peer); otherwise NCCL
    reduce-scatter / all-gather around the AdamW kernel.  Device time, max over ranks."""
    import os

    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.parallel.ddp import DistributedOptimizer, ParamBuffer

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    n = a.params * 1_000_000
    holder = torch.nn.Module()
    rows = n // 4096
    holder.w = torch.nn.Parameter(torch.zeros(rows, 4096, device="cuda", dtype=torch.bfloat16))
    arena = SymmetricArena(dist.group.WORLD) if a.fused else None
    buf = ParamBuffer(holder, shard_world=world, arena=arena, bucket_size=40_000_000)
    opt = DistributedOptimizer(buf, dist.group.WORLD, lr=1e-4, weight_decay=0.01, clip_grad=1.0, sharded=True,
                               grad_scale=1.0 / world)
    buf.grads.normal_()

    def step():
        opt.reduce_gradients()
        opt.step()

    for _ in range(3):
        step()
    dist.barrier()
    ms = _time(step, a.iters)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    _lib.check_status()
    if rank == 0:
        numel = buf.numel
        link_bytes = (world - 1) / world * numel * (4 + 2)     # fp32 gradient shards in, bf16 parameter shards out
        hbm_bytes = numel * 4 + numel / world * (30 + 4)         # zero-fill excluded: read grads, AdamW on the shard
        print(json.dumps(dict(case="dpopt", world=world, fused=bool(a.fused), params=numel, ms=float(t.item()),
                              nvlink_gbs_per_dir=link_bytes / float(t.item()) / 1e6,
                              hbm_gbs=hbm_bytes / float(t.item()) / 1e6)), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def _cp_case(a):
    """One self-attention layer of a Wan-shaped model under fused Ulysses CP = world (under torchrun on the ranks of one
    box): device time of every fused compute + exchange kernel (CUDA events around each launch, max over ranks), with
    the bytes each sends over NVLink and its roofline = max(FLOPs / measured GEMM peak, NVLink bytes / link rate)."""
    import os

    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.parallel.fused_ulysses import FusedUlysses

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    fu = FusedUlysses(SymmetricArena(dist.group.WORLD))
    H, D = a.heads, 128
    C = H * D
    S = a.seq
    S_l = (S + world - 1) // world
    fu.seq_len = S
    torch.manual_seed(rank)
    x = torch.randn(S_l, C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(3 * C, C, device="cuda") / C ** 0.5).to(torch.bfloat16).requires_grad_(True)
    b = torch.zeros(3 * C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wq = torch.ones(C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wk = torch.ones(C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    freqs = torch.randn(S_l, D // 2, 2, device="cuda")
    freqs = freqs / freqs.norm(dim=-1, keepdim=True)
    do = torch.randn(S_l, C, device="cuda", dtype=torch.bfloat16)
    L = _lib.lib()
    names = ["tt_gemm_qkv_a2a", "tt_rmsrope_fwd_scatter", "tt_attn_fwd_scatter", "tt_attn_bwd_scatter", "tt_peer_barrier"]
    events = {n: [] for n in names}

    def wrap(name):
        fn = getattr(L, name)

        def timed(*args):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            events[name].append((e0, e1))
            return rc

        setattr(L, name, timed)

    for n in names:
        wrap(n)

    def step():
        fu.begin_microbatch(fu.slab_elems(1, 1, S_l * world, C, world))
        fu.attention_qkv(x, w, b, wq, wk, freqs, 1, S_l, H, D, 1e-6).backward(do)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    for n in names:
        events[n].clear()
    for _ in range(a.iters):
        step()
    torch.cuda.synchronize()
    _lib.check_status()
    per_step = {n: sum(e0.elapsed_time(e1) for e0, e1 in ev) / a.iters for n, ev in events.items()}
    calls = {n: len(ev) // a.iters for n, ev in events.items()}
    # the same attention on this GPU without any exchange (the rank's heads over the full sequence, local tensors),
    # and with all heads over the rank's share of the work (what a data-parallel rank does in the same time share)
    Hl_own = fu.head_slots(H)[1]
    local = {}
    for tag, hh in (("own_heads", max(Hl_own, 1)), ("all_heads", H)):
        ql = torch.randn(1, S_l * world, hh, D, device="cuda", dtype=torch.bfloat16)
        kl, vl = torch.randn_like(ql), torch.randn_like(ql)
        ol, lsel = attention_fwd(ql, kl, vl)
        dol = torch.randn_like(ol)
        local[tag] = (_time(lambda: attention_fwd(ql, kl, vl), a.iters),
                      _time(lambda: attention_bwd(ql, kl, vl, ol, lsel, dol), a.iters))
        del ql, kl, vl, ol, lsel, dol
    tl = torch.tensor([x for tag in ("own_heads", "all_heads") for x in local[tag]], device="cuda", dtype=torch.float64)
    dist.all_reduce(tl, op=dist.ReduceOp.MAX)
    t = torch.tensor([per_step[n] for n in names], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        P = world
        tile = S_l * C * 2                                  # one [S_l, C] bf16 tensor
        out_frac = (P - 1) / P                              # share of a rank's rows that leaves the GPU
        Hl = (H + P - 1) // P
        attn_flops = 4.0 * Hl * (S_l * P) ** 2 * D
        rows = {
            "tt_gemm_qkv_a2a": dict(flops=2.0 * S_l * C * 3 * C, nvlink_bytes=out_frac * tile),          # V
            "tt_rmsrope_fwd_scatter": dict(flops=0.0, nvlink_bytes=3 * out_frac * tile),                  # q, k, dO
            "tt_attn_fwd_scatter": dict(flops=attn_flops, nvlink_bytes=out_frac * tile),                  # O
            "tt_attn_bwd_scatter": dict(flops=3.5 * attn_flops, nvlink_bytes=3 * out_frac * tile),        # dQ, dK, dV
            "tt_peer_barrier": dict(flops=0.0, nvlink_bytes=0.0),
        }
        out = dict(case="cp", world=world, seq=S, heads=H, rows_per_rank=S_l, kernels={})
        for i, n in enumerate(names):
            ms = float(t[i].item())
            r = rows[n]
            floor_ms = max(r["flops"] / a.peak_tflops / 1e9, r["nvlink_bytes"] / a.link_gbs / 1e6)
            out["kernels"][n] = dict(ms_per_layer=ms, launches_per_layer=calls[n], nvlink_mb=r["nvlink_bytes"] / 1e6,
                                     tflops=r["flops"] / ms / 1e9 if ms else 0.0,
                                     roofline_ms=floor_ms, fraction_of_roofline=(floor_ms / ms) if ms and floor_ms else None)
        out["local_attention_ms"] = {"own_heads_fwd": float(tl[0]), "own_heads_bwd": float(tl[1]),
                                     "all_heads_fwd_per_rank_share": float(tl[2]) / world,
                                     "all_heads_bwd_per_rank_share": float(tl[3]) / world}
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def _single_rank_fused_cases(a):
    """The fused compute + exchange kernels with a group of one (the "peer" buffers are this GPU's own), so that a
    single-process profiler run can capture them: ``qkv1`` = tt_gemm_qkv_a2a, ``ag1`` = tt_gemm2_bf16_ag,
    ``dp1`` = tt_dp_bucket_step (reduce pass and AdamW pass).  Times are CUDA events; the exchanges cost no NVLink
    bytes here, the kernels' instruction streams are the multi-rank ones."""
    dev = "cuda"
    L = _lib.lib()
    res = dict(case=a.case)
    if a.case == "qkv1":
        H, D = a.heads, 128
        C, M = H * D, a.m
        x = torch.randn(M, C, device=dev, dtype=torch.bfloat16)
        w = (torch.randn(3 * C, C, device=dev) / C ** 0.5).to(torch.bfloat16)
        b = torch.zeros(3 * C, device=dev, dtype=torch.bfloat16)
        qk = torch.empty(M, 2 * C, device=dev, dtype=torch.bfloat16)
        ssq = torch.empty(M, 2 * (C // 128), device=dev, dtype=torch.float32)
        vh = torch.empty(M * C, device=dev, dtype=torch.bfloat16)
        ptrs = (_lib.c_ll * 1)(vh.data_ptr())

        def run():
            rc = L.tt_gemm_qkv_a2a(_lib.ptr(x), _lib.c_ll(C), _lib.ptr(w), _lib.c_ll(C), _lib.ptr(b), _lib.ptr(qk),
                                   _lib.c_ll(2 * C), _lib.ptr(ssq), ptrs, _lib.c_int(1), _lib.c_int(0), _lib.c_int(M),
                                   _lib.c_int(C), _lib.c_int(C), _lib.c_int(M), _lib.c_int(H), _lib.c_int(D),
                                   _lib.ptr(_lib.status_word(torch.device(dev))), _lib.stream())
            _lib.check(rc, "tt_gemm_qkv_a2a")

        ms = _time(run, a.iters)
        ref = (x.float() @ w.float().t())
        err = (qk.float() - ref[:, :2 * C]).norm() / ref[:, :2 * C].norm()
        res.update(m=M, c=C, ms=ms, tflops=2.0 * M * C * 3 * C / ms / 1e9, rel_err_qk=float(err),
                   rel_err_ssq=float((ssq[:, :C // 128].sum(1) - qk[:, :C].float().pow(2).sum(1)).abs().max()
                                     / qk[:, :C].float().pow(2).sum(1).max()))
    elif a.case == "ag1":
        M, K, N = a.m, a.k, a.n
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
        flags = torch.zeros((M + 127) // 128, dtype=torch.int32, device=dev)
        from teletron_b200 import ops

        state = dict(epoch=0)

        def run():
            state["epoch"] += 1
            return ops.gemm_ag_gather([x.data_ptr()], M, K, w, flags, state["epoch"], 0, device=torch.device(dev))

        ms = _time(run, a.iters)
        y, _, g = run()
        ms_plain = _time(lambda: gemm(x, w), a.iters)
        res.update(m=M, n=N, k=K, ms=ms, ms_plain_gemm=ms_plain, tflops=2.0 * M * N * K / ms / 1e9,
                   gathered_ok=bool(torch.equal(g, x)), rel_err=float((y.float() - gemm(x, w).float()).norm() / y.float().norm()))
    else:  # dp1
        n = a.params * 1_000_000 // 128 * 128
        grads = torch.randn(n, device=dev)
        params = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        master, m1, v1 = (torch.zeros(n, device=dev) for _ in range(3))
        blocks = L.tt_comm_blocks()
        partial = torch.zeros(blocks, device=dev)
        gp, pp = (_lib.c_ll * 1)(grads.data_ptr()), (_lib.c_ll * 1)(params.data_ptr())

        def run(mode):
            rc = L.tt_dp_bucket_step(_lib.c_int(mode), gp, pp, _lib.c_int(1), _lib.c_int(0), _lib.c_ll(0), _lib.c_ll(n),
                                     _lib.c_ll(n), _lib.c_int(1), _lib.c_int(0), _lib.c_int(1), None, _lib.ptr(master),
                                     _lib.ptr(m1), _lib.ptr(v1), _lib.c_float(1.0), None, None, _lib.c_float(0.0), None,
                                     _lib.c_float(1e-4), _lib.c_float(0.9), _lib.c_float(0.999), _lib.c_float(1e-8),
                                     _lib.c_float(0.01), _lib.c_int(1), _lib.ptr(partial), _lib.c_int(0), _lib.stream())
            _lib.check(rc, "tt_dp_bucket_step")

        ms0 = _time(lambda: run(0), a.iters)
        ms1 = _time(lambda: run(1), a.iters)
        res.update(params=n, ms_reduce_pass=ms0, ms_adamw_pass=ms1, reduce_gbs=n * 8 / ms0 / 1e6,
                   adamw_gbs=n * (4 * 4 + 3 * 4 + 2) / ms1 / 1e6)
    _lib.check_status()
    print(json.dumps(res), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "attn", "norm", "layers", "tp", "dpopt", "cp", "qkv1", "ag1", "dp1"])
    ap.add_argument("--peak-tflops", type=float, default=1636.2, help="cp case: measured bf16 GEMM burst of the box")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="cp case: measured NVLink peer copy, GB/s per direction")
    ap.add_argument("--params", type=int, default=1400, help="dpopt case: millions of parameters")
    ap.add_argument("--inner", type=int, default=12288, help="tp case: full inner width of the MLP")
    ap.add_argument("--fused", action="store_true", help="tp case: peer-memory kernels instead of NCCL")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--m", type=int, default=32760)
    ap.add_argument("--n", type=int, default=8960)
    ap.add_argument("--k", type=int, default=1536)
    ap.add_argument("--epi", type=str, default="none", choices=["none", "gelu"])
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--kv", type=int, default=0)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--rows", type=int, default=32760)
    ap.add_argument("--c", type=int, default=1536)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    if a.case == "tp":
        return _tp_case(a)
    if a.case == "dpopt":
        return _dpopt_case(a)
    if a.case == "cp":
        return _cp_case(a)
    if a.case in ("qkv1", "ag1", "dp1"):
        return _single_rank_fused_cases(a)
    dev = "cuda"
    torch.manual_seed(0)
    res = dict(case=a.case)
    if a.case == "gemm":
        A = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device=dev, dtype=torch.bfloat16)
        B = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device=dev, dtype=torch.bfloat16)
        bias = torch.randn(a.n, device=dev, dtype=torch.bfloat16)
        out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        epi = EPI_GELU if a.epi == "gelu" else EPI_NONE
        ms = _time(lambda: gemm(A, B, a_mn=a.a_mn, b_mn=a.b_mn, bias=bias, epi=epi, out=out), a.iters)
        res.update(m=a.m, n=a.n, k=a.k, epi=a.epi, ms=ms, tflops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.case == "attn":
        kv = a.kv or a.seq
        q = torch.randn(1, a.seq, a.heads, 128, device=dev, dtype=torch.bfloat16)
        k = torch.randn(1, kv, a.heads, 128, device=dev, dtype=torch.bfloat16)
        v = torch.randn(1, kv, a.heads, 128, device=dev, dtype=torch.bfloat16)
        o, lse = attention_fwd(q, k, v)
        flops = 4.0 * a.heads * a.seq * kv * 128
        if a.bwd:
            do = torch.randn_like(o)
            ms = _time(lambda: attention_bwd(q, k, v, o, lse, do), a.iters)
            res.update(seq=a.seq, kv=kv, heads=a.heads, bwd=True, ms=ms, tflops_at_2p5x=2.5 * flops / ms / 1e9,
                       tflops_executed=3.5 * flops / ms / 1e9)
        else:
            ms = _time(lambda: attention_fwd(q, k, v), a.iters)
            res.update(seq=a.seq, kv=kv, heads=a.heads, bwd=False, ms=ms, tflops=flops / ms / 1e9)
    elif a.case == "layers":
        from teletron_b200.models import WanModel, wan_config
        from teletron_b200.parallel.ddp import ParamBuffer
        from teletron_b200.ops.flow import flow_mse

        model = WanModel(wan_config("wan2.1-1.3b-t2v", num_layers=a.layers)).to(dev).to(torch.bfloat16).train()
        buf = ParamBuffer(model)
        x0 = torch.randn(1, 16, 21, 60, 104, device=dev, dtype=torch.bfloat16)
        nz = torch.randn_like(x0)
        ctx = torch.randn(1, 512, 4096, device=dev, dtype=torch.bfloat16)
        t = torch.tensor([500.0], device=dev)

        def step():
            buf.zero_grads()
            flow_mse(model(0.5 * x0 + 0.5 * nz, t, ctx), x0, nz).backward()

        ms = _time(step, a.iters)
        res.update(layers=a.layers, ms=ms, launches_per_step=None)
    else:
        x = torch.randn(a.rows, a.c, device=dev, dtype=torch.bfloat16)
        mod = torch.randn(1, 6, a.c, device=dev)
        ms = _time(lambda: adaln(x, mod[:, 1], mod[:, 0], a.rows), a.iters)
        res.update(rows=a.rows, c=a.c, ms=ms, gbps=2.0 * a.rows * a.c * 2 / ms / 1e6)
    _lib.check_status()
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
