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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "attn", "norm", "layers", "tp", "dpopt"])
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
