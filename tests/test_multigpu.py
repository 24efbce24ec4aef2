"""Multi-GPU tests (need >= 2 GPUs in one box): peer-memory fused optimizer step vs the NCCL path,
Ulysses context parallelism through the CUDA kernels vs one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from dist_utils import run_distributed

needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
needs4 = pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
needs8 = pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return (0.5 * (a - b).norm() / (a.norm() + b.norm() + 1e-30)).item()


def _opt_worker(rank, world, fused, clip, overlap=False):
    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.ops import _lib
    from teletron_b200.parallel.ddp import DistributedOptimizer, ParamBuffer

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.Linear(512, 264),
                                torch.nn.Linear(264, 520)).cuda().to(torch.bfloat16)
    arena = SymmetricArena(dist.group.WORLD) if fused else None
    buf = ParamBuffer(model, shard_world=world, arena=arena, bucket_size=50_000)   # several buckets, ragged last one
    assert len(buf.buckets) >= 6
    opt = DistributedOptimizer(buf, dist.group.WORLD, lr=1e-2, weight_decay=0.1, clip_grad=clip, sharded=True,
                               grad_scale=1.0 / world, overlap=overlap)
    assert opt.fused == fused
    norms = []
    for step in range(3):
        opt.zero_grad()
        g = torch.Generator(device="cuda").manual_seed(100 * step + rank)
        buf.grads.copy_(torch.randn(buf.numel, device="cuda", generator=g))
        if overlap:      # what the gradient-ready hooks of a backward pass do, in backward order
            opt.begin_last_microbatch()
            for name, p in reversed(buf.named):
                p.grad_ready()
            assert opt.fired_in_backward == len(buf.buckets)
        opt.reduce_gradients()
        _, n, _ = opt.step()
        norms.append(float(n))
    torch.cuda.synchronize()
    _lib.check_status()
    full = opt.gather_full_state()
    return buf.params.float().cpu(), (full["master"] if full is not None else None), norms


def _check_fused_optimizer(world, clip):
    ref = run_distributed(_opt_worker, world, False, clip, backend="nccl")
    got = run_distributed(_opt_worker, world, True, clip, backend="nccl")
    over = run_distributed(_opt_worker, world, True, clip, True, backend="nccl")
    for r in range(world):
        assert torch.equal(got[r][0], got[0][0])                      # replicas agree bit for bit
        assert rel(got[r][0], ref[r][0]) < 1e-3                          # bf16 params
        assert all(abs(a - b) < 1e-3 * abs(b) for a, b in zip(got[r][2], ref[r][2]))
        # reductions started bucket by bucket on the side stream: not one bit differs
        assert torch.equal(over[r][0], got[r][0]) and over[r][2] == got[r][2]
    assert rel(got[0][1], ref[0][1]) < 1e-5                              # fp32 master weights, whole buffer
    assert torch.equal(over[0][1], got[0][1])


@needs2
@pytest.mark.parametrize("clip", [0.0, 1.0])
def test_fused_dp_optimizer_matches_nccl(clip):
    _check_fused_optimizer(2, clip)


@needs8
@pytest.mark.parametrize("clip", [0.0, 1.0])
def test_fused_dp_optimizer_matches_nccl_with_eight_peers(clip):
    _check_fused_optimizer(8, clip)


# shapes for the context-parallel tests: (hidden, heads, latent f, h, w) -> f * h/2 * w/2 tokens
SMALL = (256, 2, 3, 16, 20)            # 240 tokens: below the CTA-pair GEMM's row minimum (copy-kernel exchange of V)
RAGGED = (512, 4, 3, 34, 42)           # 1,071 tokens: not a multiple of 2, 4 or 8 -> padded tail masked by key length
UNEVEN = (384, 3, 3, 34, 42)           # 3 heads: do not divide by 2 or 4
WAN13_HEADS = (1536, 12, 3, 34, 42)    # the 1.3B model's 12 heads (CP = 8: two head slots per rank, two ranks idle)


def _cp_worker(rank, world, fused=False, layers=2, recompute_layers=0, shape=SMALL):
    from teletron_b200 import ops
    from teletron_b200.models import WanModel, wan_config
    from teletron_b200.ops import _lib
    from teletron_b200.parallel import state as mpu
    from teletron_b200.parallel.ulysses import UlyssesContext

    mpu.initialize_model_parallel(context_parallel_size=world)
    cp = UlyssesContext(mpu.get_context_parallel_group(), world, rank)
    if fused:
        from teletron_b200.dist import SymmetricArena
        from teletron_b200.parallel.fused_ulysses import FusedUlysses

        cp.fused = FusedUlysses(SymmetricArena(mpu.get_context_parallel_group()))
        cp.fused.poison = True      # NaN-filled peer buffers: a read before arrival would show in the comparison
    torch.manual_seed(0)
    extra = dict(recompute_granularity="full", recompute_method="block",
                 recompute_num_layers=recompute_layers) if recompute_layers else {}
    dim, heads, lf, lh, lw = shape
    cfg = wan_config("wan-tiny", dim=dim, num_heads=heads, ffn_dim=512, text_dim=64, freq_dim=64, num_layers=layers,
                     **extra)
    model = WanModel(cfg, cp).cuda().to(torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 16, lf, lh, lw, generator=g).cuda().bfloat16()
    ctx = torch.randn(1, 40, 64, generator=g).cuda().bfloat16()
    t = torch.tensor([400.0]).cuda()
    for _ in range(2 if fused else 1):  # twice: the slab and staging buffers are recycled
        model.zero_grad(set_to_none=True)
        out = model(x, t, ctx)
        out.float().square().mean().backward()
    grads = {n: p.grad.float() for n, p in model.named_parameters() if p.grad is not None}
    for v in grads.values():
        torch.distributed.all_reduce(v)
    torch.cuda.synchronize()
    _lib.check_status()
    return out.float().cpu(), {k: v.cpu() for k, v in grads.items()}


def _single_gpu_reference(layers=2, shape=SMALL):
    from teletron_b200.models import WanModel, wan_config

    torch.manual_seed(0)
    dim, heads, lf, lh, lw = shape
    cfg = wan_config("wan-tiny", dim=dim, num_heads=heads, ffn_dim=512, text_dim=64, freq_dim=64, num_layers=layers)
    model = WanModel(cfg).cuda().to(torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 16, lf, lh, lw, generator=g).cuda().bfloat16()
    ctx = torch.randn(1, 40, 64, generator=g).cuda().bfloat16()
    t = torch.tensor([400.0]).cuda()
    out = model(x, t, ctx)
    out.float().square().mean().backward()
    return out.float().cpu(), {n: p.grad.float().cpu() for n, p in model.named_parameters() if p.grad is not None}


@needs2
@pytest.mark.parametrize("fused", [False, True])
def test_ulysses_cp2_matches_single_gpu(fused):
    ref_out, ref_g = _single_gpu_reference()
    outs = run_distributed(_cp_worker, 2, fused, backend="nccl")
    for out, grads in outs:
        assert rel(out, ref_out) < 1e-3          # same threshold as the reference's model test
        bad = [(n, rel(grads[n], ref_g[n])) for n in ref_g if ref_g[n].norm() > 2e-4 and rel(grads[n], ref_g[n]) > 2e-2]
        assert not bad, bad


def _check_cp(world, shape, fused=True):
    ref_out, ref_g = _single_gpu_reference(shape=shape)
    outs = run_distributed(_cp_worker, world, fused, 2, 0, shape, backend="nccl")
    for out, grads in outs:
        assert rel(out, ref_out) < 1e-3
        assert (out - ref_out).abs().max() < 0.05 * ref_out.abs().max()
        bad = [(n, rel(grads[n], ref_g[n])) for n in ref_g if ref_g[n].norm() > 2e-4 and rel(grads[n], ref_g[n]) > 2e-2]
        assert not bad, bad


@needs2
@pytest.mark.parametrize("shape", [RAGGED, UNEVEN], ids=["ragged-qkv-epilogue", "three-heads"])
def test_fused_ulysses_cp2_ragged_tokens_and_uneven_heads(shape):
    """RAGGED: 536 rows per rank, so the q/k/v projection runs as the GEMM whose epilogue stores V into the head
    owner and hands the row statistics to the norm kernel; 1,071 tokens leave one padded key that the attention
    kernel masks.  UNEVEN: three heads over two ranks (two head slots each, the second rank owns one head)."""
    _check_cp(2, shape)


@needs4
@pytest.mark.parametrize("shape", [RAGGED, UNEVEN], ids=["ragged", "three-heads-one-rank-idle"])
def test_fused_ulysses_cp4(shape):
    _check_cp(4, shape)


@needs8
@pytest.mark.parametrize("shape", [WAN13_HEADS], ids=["twelve-heads"])
def test_fused_ulysses_cp8(shape):
    _check_cp(8, shape)


def _dp_cp_trainer_worker(rank, world, cp, fused):
    """Two optimizer steps of a small Wan DiT through the Trainer on a fixed global batch of 4 samples (data, noise
    and timestep are functions of the sample index), in any DP x CP layout."""
    import os

    from teletron_b200.data import SyntheticLatentDataset
    from teletron_b200.ops import _lib
    from teletron_b200.parallel import state as mpu
    from teletron_b200.train import Trainer, make_forward_step, parse_args

    os.environ["WORLD_SIZE"], os.environ["RANK"], os.environ["LOCAL_RANK"] = str(world), str(rank), str(rank)
    argv = (f"--model ParallelWanModel --model-preset wan-tiny --hidden-size 512 --num-attention-heads 4 "
            f"--ffn-hidden-size 1024 --num-layers 2 --bf16 --train-iters 100 --micro-batch-size 1 --global-batch-size 4 "
            f"--lr 1e-3 --num-frames 9 --video-resolution 272 336 --log-interval 1000 --clip-grad 1.0 --seed 5 "
            f"--synthetic-latents --context-parallel-size {cp} --fused-comm {'on' if fused else 'off'} "
            f"--ddp-bucket-size 300000" + (" --use-distributed-optimizer" if world > 1 else "")).split()
    a = parse_args(argv=argv)
    t = Trainer(a, build_data=False)
    ds = SyntheticLatentDataset(9, 272, 336, text_len=32, text_dim=64, seed=7, fixed_noise=True)   # 3*17*21 = 1,071 tokens
    d = mpu.get_data_parallel_rank() if world > 1 else 0
    n_mb = a.num_micro_batches
    pool = [{k: v.unsqueeze(0).cuda() for k, v in ds[i].items()} for i in range(d * n_mb, (d + 1) * n_mb)]
    fwd = make_forward_step()
    losses, norms = [], []
    for _ in range(2):
        ld, _, gn, _ = t.train_step(fwd, iter(pool))
        losses.append(float(ld["loss"]))
        norms.append(float(gn))
    torch.cuda.synchronize()
    _lib.check_status()
    return losses, norms, t.buffer.params[:200000].float().cpu(), bool(t.optimizer.overlap), t.optimizer.fired_in_backward


def _check_trainer_layout(world, cp):
    (l1, n1, p1, _, _), = run_distributed(_dp_cp_trainer_worker, 1, 1, False, backend="nccl")
    outs = run_distributed(_dp_cp_trainer_worker, world, cp, True, backend="nccl")
    for losses, norms, params, overlap, fired in outs:
        assert overlap and fired > 0                       # bucket reductions started from the backward hooks
        assert all(abs(a - b) < 2e-3 * abs(b) for a, b in zip(losses, l1)), (losses, l1)
        assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(norms, n1)), (norms, n1)
        assert torch.equal(params, outs[0][2])
        assert rel(params, p1) < 2e-3


@needs2
def test_trainer_cp2_fused_matches_one_gpu():
    _check_trainer_layout(2, 2)


@needs4
def test_trainer_dp2_cp2_fused_matches_one_gpu():
    _check_trainer_layout(4, 2)


@needs8
def test_trainer_dp2_cp4_fused_matches_one_gpu():
    _check_trainer_layout(8, 4)


@needs2
def test_ulysses_cp2_fused_with_recompute_recycles_the_slab():
    """Four layers, the first three checkpointed: the symmetric slab is sized for three layers, so the run
    only fits (and only matches) when discarded forward passes hand their regions back."""
    ref_out, ref_g = _single_gpu_reference(layers=4)
    outs = run_distributed(_cp_worker, 2, True, 4, 3, backend="nccl")
    for out, grads in outs:
        assert rel(out, ref_out) < 1e-3
        bad = [(n, rel(grads[n], ref_g[n])) for n in ref_g if ref_g[n].norm() > 2e-4 and rel(grads[n], ref_g[n]) > 2e-2]
        assert not bad, bad


def _tp_worker(rank, world, fused):
    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.ops import _lib
    from teletron_b200.parallel.tp import ColumnParallelLinear, FusedTP, RowParallelLinear, TPContext

    torch.manual_seed(0)
    tp = TPContext(dist.group.WORLD, world, rank)
    if fused:
        tp.fused = FusedTP(SymmetricArena(dist.group.WORLD))
    rows, C, inner = 200, 256, 768            # 200 rows per rank: not a multiple of the 128-row tile
    col = ColumnParallelLinear(C, inner, tp).cuda().to(torch.bfloat16)
    row = RowParallelLinear(inner, C, tp).cuda().to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(7)
    x_full = torch.randn(world * rows, C, device="cuda", generator=g).to(torch.bfloat16)
    dy_full = torch.randn(world * rows, C, device="cuda", generator=g).to(torch.bfloat16)
    x = x_full[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    outs = []
    for _ in range(3):                        # three rounds: the peer buffers are double-buffered
        x.grad = None
        col.zero_grad()
        row.zero_grad()
        y = row(col(x, act="gelu"))
        y.backward(dy_full[rank * rows:(rank + 1) * rows])
        outs = [y.detach(), x.grad, col.weight.grad, col.bias.grad, row.weight.grad]
    if fused:
        # the gathering GEMM kernel (400 gathered rows, 384 columns) against the variant whose TMA loads read the peers
        from teletron_b200 import ops

        xd = x.detach()
        y1, _, g1 = tp.fused.ag_gemm(xd, col.weight.detach(), bias=col.bias.detach())
        buf = tp.fused._x[tp.fused._n_ag & 1]
        y2 = ops.gemm_ag(buf.peer_ptrs, rows, C, col.weight.detach(), bias=col.bias.detach(), device=xd.device)
        torch.cuda.synchronize()
        assert g1 is not None and torch.equal(g1, x_full), "the kernel's gathered operand is not the all-gather"
        assert rel(y1, y2) < 1e-3, rel(y1, y2)
    torch.cuda.synchronize()
    _lib.check_status()
    return [o.float().cpu() for o in outs]


@needs2
def test_fused_tp_linears_match_nccl():
    ref = run_distributed(_tp_worker, 2, False, backend="nccl")
    got = run_distributed(_tp_worker, 2, True, backend="nccl")
    for r in range(2):
        for a, b in zip(got[r], ref[r]):
            assert rel(a, b) < 4e-3


def _hy_inputs():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 16, 4, 16, 16, generator=g)             # 4 * 8 * 8 = 256 video tokens
    text = torch.randn(1, 24, 64, generator=g)
    mask = torch.ones(1, 24, dtype=torch.long)
    mask[:, 17:] = 0
    return x, torch.tensor([700.0]), text, mask, torch.randn(1, 32, generator=g), torch.tensor([6000.0])


def _hy_run(m):
    x, t, text, mask, pooled, guid = _hy_inputs()
    out = m(x.cuda().bfloat16(), t.cuda(), text.cuda().bfloat16(), mask.cuda(), pooled.cuda().bfloat16(), guid.cuda())
    out.float().square().mean().backward()
    torch.cuda.synchronize()
    return out.detach().float().cpu(), {n: p.grad.detach().float().cpu() for n, p in m.named_parameters()
                                        if p.grad is not None}


def _hy_tp_worker(rank, world, full_sd, fused):
    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.models.hunyuan import HunyuanVideoModel, hunyuan_config
    from teletron_b200.ops import _lib
    from teletron_b200.parallel.tp import FusedTP, TPContext, tp_shard_dims, tp_shard_state_dict

    tp = TPContext(dist.group.WORLD, world, rank)
    if fused:
        tp.fused = FusedTP(SymmetricArena(dist.group.WORLD))
    m = HunyuanVideoModel(hunyuan_config("hunyuan-tiny"), None, tp)
    m.load_state_dict(tp_shard_state_dict(full_sd, tp_shard_dims(m), rank, world))
    dims = tp_shard_dims(m, params=True)
    m = m.cuda().to(torch.bfloat16)
    out, grads = _hy_run(m)
    for n, g in grads.items():
        if n not in dims:                       # replicated parameters see only this rank's rows
            gg = g.cuda()
            dist.all_reduce(gg)
            grads[n] = gg.cpu()
    _lib.check_status()
    return out, grads


@needs2
@pytest.mark.parametrize("fused", [False, True])
def test_hunyuan_tp2_matches_single_gpu(fused):
    import copy

    from teletron_b200.models.hunyuan import HunyuanVideoModel, hunyuan_config
    from teletron_b200.parallel.tp import TPContext, tp_merge_state_dicts, tp_shard_dims

    torch.manual_seed(0)
    ref = HunyuanVideoModel(hunyuan_config("hunyuan-tiny"))
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    full_sd = {k: v.clone() for k, v in ref.state_dict().items()}
    ref_out, ref_g = _hy_run(copy.deepcopy(ref).cuda().to(torch.bfloat16))
    outs = run_distributed(_hy_tp_worker, 2, full_sd, fused, backend="nccl")
    dims = tp_shard_dims(HunyuanVideoModel(hunyuan_config("hunyuan-tiny"), None, TPContext(None, 2, 0)), params=True)
    merged = tp_merge_state_dicts([o[1] for o in outs], dims)
    for out, _ in outs:
        assert rel(out, ref_out) < 1e-2
    bad = [(n, rel(merged[n], g)) for n, g in ref_g.items() if g.norm() > 2e-4 and rel(merged[n], g) > 3e-2]
    assert not bad, bad


def _hy_cp_worker(rank, world, full_sd, tp_size, fused):
    """HunyuanVideo (1 dual + 2 single blocks) under TP x CP; gradients summed the way the optimizer's reductions do."""
    import torch.distributed as dist

    from teletron_b200.dist import SymmetricArena
    from teletron_b200.models.hunyuan import HunyuanVideoModel, hunyuan_config
    from teletron_b200.ops import _lib
    from teletron_b200.parallel import state as mpu
    from teletron_b200.parallel.fused_ulysses import FusedUlysses
    from teletron_b200.parallel.tp import FusedTP, TPContext, tp_shard_dims, tp_shard_state_dict
    from teletron_b200.parallel.ulysses import UlyssesContext

    cp_size = world // tp_size
    mpu.initialize_model_parallel(tensor_model_parallel_size=tp_size, context_parallel_size=cp_size)
    tp = TPContext(mpu.get_tensor_model_parallel_group(), tp_size, mpu.get_tensor_model_parallel_rank())
    cp = UlyssesContext(mpu.get_context_parallel_group(), cp_size, mpu.get_context_parallel_rank())
    if fused:
        cp.fused = FusedUlysses(SymmetricArena(mpu.get_context_parallel_group()))
        if tp_size > 1:
            tp.fused = FusedTP(SymmetricArena(mpu.get_tensor_model_parallel_group()))
    cfg = hunyuan_config("hunyuan-tiny", hidden_size=512, num_attention_heads=4)
    m = HunyuanVideoModel(cfg, cp, tp)
    m.load_state_dict(tp_shard_state_dict(full_sd, tp_shard_dims(m), tp.rank, tp_size))
    dims = tp_shard_dims(m, params=True)
    m = m.cuda().to(torch.bfloat16)
    for _ in range(2):                          # twice: slab and staging buffers are recycled
        m.zero_grad(set_to_none=True)
        out, grads = _hy_run(m)
    for n, g in grads.items():
        gg = g.cuda()
        # sharded parameters: partial sums over the CP group; replicated ones: over TP x CP
        dist.all_reduce(gg, group=mpu.get_context_parallel_group() if n in dims else None)
        grads[n] = gg.cpu()
    _lib.check_status()
    return out, grads, mpu.get_tensor_model_parallel_rank()


def _check_hunyuan_layout(world, tp_size):
    import copy

    from teletron_b200.models.hunyuan import HunyuanVideoModel, hunyuan_config
    from teletron_b200.parallel.tp import TPContext, tp_merge_state_dicts, tp_shard_dims

    torch.manual_seed(0)
    cfg = hunyuan_config("hunyuan-tiny", hidden_size=512, num_attention_heads=4)
    ref = HunyuanVideoModel(cfg)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    full_sd = {k: v.clone() for k, v in ref.state_dict().items()}
    ref_out, ref_g = _hy_run(copy.deepcopy(ref).cuda().to(torch.bfloat16))
    outs = run_distributed(_hy_cp_worker, world, full_sd, tp_size, True, backend="nccl")
    dims = tp_shard_dims(HunyuanVideoModel(cfg, None, TPContext(None, tp_size, 0)), params=True)
    by_tp = {}
    for out, grads, tpr in outs:
        assert rel(out, ref_out) < 1e-2
        by_tp.setdefault(tpr, grads)
    merged = tp_merge_state_dicts([by_tp[r] for r in range(tp_size)], dims)
    bad = [(n, rel(merged[n], g)) for n, g in ref_g.items() if g.norm() > 2e-4 and rel(merged[n], g) > 3e-2]
    assert not bad, bad


@needs2
def test_hunyuan_cp2_fused_joint_attention_matches_single_gpu():
    """Video q / k / v reach the head owners through the norm kernel's stores, the text tokens sit behind them in
    the same buffers, the padded text tail is masked by key length, outputs return through the attention epilogue."""
    _check_hunyuan_layout(2, 1)


@needs4
def test_hunyuan_tp2_cp2_fused_matches_single_gpu():
    _check_hunyuan_layout(4, 2)


def _encoder_fed_nccl_worker(rank, world):
    """Rank 0 trains a two-layer DiT, rank 1 is its encoder rank; samples cross over NCCL send / recv."""
    import os

    from teletron_b200.ops import _lib
    from teletron_b200.train import Trainer, make_forward_step, parse_args

    os.environ["WORLD_SIZE"], os.environ["RANK"] = str(world), str(rank)
    argv = ("--model ParallelWanModel --model-preset wan-tiny --hidden-size 256 --num-attention-heads 2 "
            "--ffn-hidden-size 512 --num-layers 2 --bf16 --train-iters 3 --micro-batch-size 1 --lr 1e-3 "
            "--num-frames 5 --video-resolution 64 64 --log-interval 100 --clip-grad 1.0 --seed 5 "
            "--distributed-backend nccl --distributed-vae --distributed-vae-world-size 1 "
            "--encoder-name synthetic_wan_encoder --dataset-type FakeDataset").split()

    def extra_args(p):
        p.add_argument("--encoder-name", type=str, default=None)
        p.add_argument("--text-dim", type=int, default=64)
        p.add_argument("--text-len", type=int, default=16)
        return p

    a = parse_args(extra_args, argv)
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    before = t.buffer.params.float().clone()
    t.pretrain(make_forward_step())
    torch.cuda.synchronize()
    _lib.check_status()
    return a.iteration, float((t.buffer.params.float() - before).abs().sum())


@needs2
def test_training_fed_by_an_encoder_rank_over_nccl():
    outs = run_distributed(_encoder_fed_nccl_worker, 2, backend="nccl", timeout=150)
    assert outs[1] == "encoder-rank-done"
    iters, moved = outs[0]
    assert iters == 3 and moved > 0


def _ckpt_nccl_worker(rank, world, root, mode, backend="nccl"):
    """DP2 with the sharded optimizer on the peer-memory path: "full" = three steps; "save" = two steps and a
    checkpoint; "resume" = load it and take the third step."""
    import os

    from teletron_b200.ops import _lib
    from teletron_b200.train import Trainer, make_forward_step, parse_args

    os.environ["WORLD_SIZE"], os.environ["RANK"] = str(world), str(rank)
    argv = ("--model ParallelWanModel --model-preset wan-tiny --hidden-size 256 --num-attention-heads 2 "
            "--ffn-hidden-size 512 --num-layers 2 --train-iters 3 --micro-batch-size 1 --global-batch-size 2 "
            "--lr 1e-3 --num-frames 5 --video-resolution 64 64 --log-interval 100 --clip-grad 1.0 --seed 5 "
            f"--distributed-backend {backend} --use-distributed-optimizer --synthetic-latents --ddp-bucket-size 20000 "
            f"--save {root}/{'full' if mode == 'full' else 'run'}").split()
    if backend == "nccl":
        argv.append("--bf16")
    if mode == "resume":
        argv += ["--load", f"{root}/run"]

    def extra_args(p):
        p.add_argument("--text-dim", type=int, default=64)
        p.add_argument("--text-len", type=int, default=16)
        return p

    a = parse_args(extra_args, argv)
    t = Trainer(a)
    start = a.iteration
    for it in range(start, 2 if mode == "save" else 3):
        g = torch.Generator().manual_seed(100 + it)     # the timestep stream is a function of the iteration
        t.train_step(make_forward_step(timestep_generator=g))
        a.iteration = it + 1
        a.consumed_train_samples += a.global_batch_size
    if mode == "save":
        t.save(2)
    if backend == "nccl":
        torch.cuda.synchronize()
        _lib.check_status()
    full = t.optimizer.gather_full_state()
    return start, t.buffer.params.float().cpu(), None if full is None else full["exp_avg_sq"]


@needs2
def test_sharded_optimizer_checkpoint_round_trip_over_nccl(tmp_path):
    """The optimizer shares travel to rank 0 bucket by bucket (``gather`` over NCCL), the file is memory-mapped
    on load, and the resumed run continues bit for bit."""
    full = run_distributed(_ckpt_nccl_worker, 2, str(tmp_path), "full", backend="nccl", timeout=150)
    run_distributed(_ckpt_nccl_worker, 2, str(tmp_path), "save", backend="nccl", timeout=150)
    res = run_distributed(_ckpt_nccl_worker, 2, str(tmp_path), "resume", backend="nccl", timeout=150)
    assert res[0][0] == 2 and full[0][0] == 0
    assert torch.equal(res[0][1], full[0][1]) and torch.equal(res[1][1], full[1][1])
    assert torch.equal(res[0][2], full[0][2]) and float(full[0][2].abs().sum()) > 0
