"""HunyuanVideo DiT on CPU (fp32): key-length masking vs a dense boolean mask, and context /
tensor parallel runs (gloo) against the single-rank model — output and every parameter gradient."""
import pytest
import torch

from dist_utils import run_distributed
from teletron_b200 import ops
from teletron_b200.models.hunyuan import HunyuanVideoModel, hunyuan_config, joint_attention
from teletron_b200.parallel import state as mpu
from teletron_b200.parallel.tp import TPContext, tp_merge_state_dicts, tp_shard_dims, tp_shard_state_dict
from teletron_b200.parallel.ulysses import UlyssesContext


def _cfg():
    return hunyuan_config("hunyuan-tiny", hidden_size=64, num_attention_heads=4, attention_head_dim=16,
                          rope_axes_dim=(4, 6, 6))


def _inputs():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 16, 2, 8, 8, generator=g)            # 2*4*4 = 32 video tokens
    text = torch.randn(1, 12, 64, generator=g)
    mask = torch.ones(1, 12, dtype=torch.long)
    mask[:, 9:] = 0
    return x, torch.tensor([700.0]), text, mask, torch.randn(1, 32, generator=g), torch.tensor([6000.0])


def test_key_length_mask_equals_dense_mask():
    g = torch.Generator().manual_seed(1)
    S, T, H, D = 20, 6, 2, 8
    qv, kv, vv = (torch.randn(1, S, H, D, generator=g) for _ in range(3))
    qt, kt, vt = (torch.randn(1, T, H, D, generator=g) for _ in range(3))
    lens = torch.tensor([4])
    ov, ot = joint_attention(qv, kv, vv, qt, kt, vt, None, lens)
    q, k, v = (torch.cat(p, 1).transpose(1, 2) for p in ((qv, qt), (kv, kt), (vv, vt)))
    n = S + 4
    dense = torch.zeros(1, 1, S + T, S + T, dtype=torch.bool)
    dense[:, :, :n, :n] = True                    # the reference's mask (hunyuan/model.py:318-342)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=dense).transpose(1, 2)
    assert (ov - ref[:, :S]).abs().max() < 1e-5
    assert (ot[:, :4] - ref[:, S:n]).abs().max() < 1e-5   # valid text queries agree; padded rows are unused


def _run(model):
    out = model(*_inputs())
    out.square().mean().backward()
    return out.detach(), {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}


def _single():
    torch.manual_seed(0)
    m = HunyuanVideoModel(_cfg())
    return m, _run(m)


def _cp_worker(rank, world):
    mpu.initialize_model_parallel(context_parallel_size=world)
    torch.manual_seed(0)
    m = HunyuanVideoModel(_cfg(), UlyssesContext(mpu.get_context_parallel_group(), world, rank))
    out, grads = _run(m)
    for g in grads.values():
        torch.distributed.all_reduce(g)            # every parameter gradient is a partial sum over CP
    return out, grads


def test_context_parallel_matches_single_rank():
    _, (ref_out, ref_g) = _single()
    for out, grads in run_distributed(_cp_worker, 2):
        assert (out - ref_out).abs().max() < 1e-5
        for n, g in ref_g.items():
            assert (grads[n] - g).norm() <= 1e-4 * (g.norm() + 1e-6), n


def _tp_worker(rank, world, full_sd):
    mpu.initialize_model_parallel(tensor_model_parallel_size=world)
    tp = TPContext(mpu.get_tensor_model_parallel_group(), world, rank)
    m = HunyuanVideoModel(_cfg(), None, tp)
    m.load_state_dict(tp_shard_state_dict(full_sd, tp_shard_dims(m), rank, world))   # state-dict names
    pdims = tp_shard_dims(m, params=True)                                           # parameter names
    out, grads = _run(m)
    for n, g in grads.items():
        if n not in pdims:
            torch.distributed.all_reduce(g)        # replicated parameters see only this rank's rows
    return out, grads, m.state_dict()


def test_tensor_parallel_matches_single_rank_and_shards_round_trip():
    m, (ref_out, ref_g) = _single()
    full_sd = {k: v.clone() for k, v in m.state_dict().items()}
    outs = run_distributed(_tp_worker, 2, full_sd)
    probe = HunyuanVideoModel(_cfg(), None, TPContext(None, 2, 0))
    merged_g = tp_merge_state_dicts([o[1] for o in outs], tp_shard_dims(probe, params=True))
    merged_sd = tp_merge_state_dicts([o[2] for o in outs], tp_shard_dims(probe))
    assert any(k.endswith("attn.to_q.weight") for k in full_sd) and not any("to_qkv" in k for k in full_sd)
    for out, _, _ in outs:
        assert (out - ref_out).abs().max() < 1e-5
    for n, g in ref_g.items():
        assert (merged_g[n] - g).norm() <= 1e-4 * (g.norm() + 1e-6), n
    for k, v in full_sd.items():
        assert torch.equal(merged_sd[k], v), k


def _hy_train_args(world, extra=""):
    import os

    from teletron_b200.train import parse_args

    os.environ["WORLD_SIZE"], os.environ["RANK"] = str(world), os.environ.get("RANK", "0")
    argv = (f"--model ParallelHunyuanVideoModel --model-preset hunyuan-tiny --train-iters 2 --micro-batch-size 1 "
            f"--global-batch-size 2 --lr 1e-3 --synthetic-latents --num-frames 5 --video-resolution 64 64 "
            f"--log-interval 100 --clip-grad 1.0 --seed 11 --distributed-backend gloo {extra}").split()

    def extra_args(p):
        p.add_argument("--text-len", type=int, default=12)
        return p

    return parse_args(extra_args, argv)


def _hy_train_worker(rank, world, extra):
    from teletron_b200.train import Trainer, make_hunyuan_forward_step

    t = Trainer(_hy_train_args(world, extra))
    gen = torch.Generator().manual_seed(4)
    fwd = make_hunyuan_forward_step(timestep_generator=gen)
    losses = []
    for _ in range(2):
        ld, skipped, gnorm, _ = t.train_step(fwd)
        assert skipped == 0 and torch.isfinite(gnorm)
        losses.append(float(ld["loss"]))
    return losses, t.buffer.params.float().clone()


def test_hunyuan_trains_through_the_trainer_alone_and_with_cp2_tp2():
    """Same seed, data and timesteps: one rank and Ulysses CP = 2 give the same loss (the noise is drawn on the
    source rank of the TP x CP group and broadcast; its generator state equals the one-rank state).  Under TP = 2
    the sharded layers draw their initial weights per shard, so only agreement between the ranks is checked."""
    (single, p1), = run_distributed(_hy_train_worker, 1, "")
    assert all(l == l and l > 0 for l in single)
    cp = run_distributed(_hy_train_worker, 2, "--context-parallel-size 2 --use-distributed-optimizer")
    assert cp[0][0] == cp[1][0] and torch.equal(cp[0][1], cp[1][1])
    assert abs(cp[0][0][0] - single[0]) < 2e-3 * abs(single[0])
    tp = run_distributed(_hy_train_worker, 2, "--tensor-model-parallel-size 2")
    assert tp[0][0] == tp[1][0] and all(l == l and l > 0 for l in tp[0][0])


def test_hunyuan_i2v_step_builds_the_33_channel_input():
    from teletron_b200.data import SyntheticHunyuanDataset
    from teletron_b200.models.hunyuan import ParallelHunyuanVideoModel
    from teletron_b200.train import make_hunyuan_forward_step

    cfg = hunyuan_config("hunyuan-tiny", in_channels=33)
    model = ParallelHunyuanVideoModel(cfg)
    ds = SyntheticHunyuanDataset(5, 64, 64, text_len=12, text_dim=cfg.text_embed_dim,
                                 pooled_dim=cfg.pooled_projection_dim, i2v=True, dtype=torch.float32)
    item = ds[3]
    assert item["first_ref_image"].shape == (16, 1, 8, 8) and 3 <= int(item["prompt_mask"].sum()) <= 12
    batch = {k: v.unsqueeze(0) for k, v in item.items()}
    seen = {}
    hook = model.x_embedder.register_forward_pre_hook(lambda m, a: seen.setdefault("x", a[0]))
    orig = model.patchify

    def spy(x):
        seen["in"] = x
        return orig(x)

    model.patchify = spy
    loss, loss_func = make_hunyuan_forward_step()(iter([batch]), model)
    hook.remove()
    assert seen["in"].shape[1] == 33
    x = seen["in"]
    assert torch.equal(x[:, 16:32, :1], batch["first_ref_image"]) and float(x[:, 16:32, 1:].abs().sum()) == 0
    assert float(x[:, 32, 0].min()) == 1.0 and float(x[:, 32, 1:].abs().sum()) == 0
    loss.backward()
    _, reduced = loss_func(loss)
    assert torch.isfinite(reduced["loss"])


def _hy_encoder_fed_worker(rank, world):
    from teletron_b200.train import Trainer, make_hunyuan_forward_step

    a = _hy_train_args(world, "--distributed-vae --distributed-vae-world-size 1 --dataset-type FakeDataset")
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    before = t.buffer.params.float().clone()
    t.pretrain(make_hunyuan_forward_step())
    return float((t.buffer.params.float() - before).abs().sum())


def test_hunyuan_training_fed_by_an_encoder_rank():
    outs = run_distributed(_hy_encoder_fed_worker, 2, timeout=240)
    assert outs[1] == "encoder-rank-done" and outs[0] > 0


def _hy_tp_resume_worker(rank, world, root, mode):
    import os

    from teletron_b200.train import Trainer, make_hunyuan_forward_step

    extra = f"--tensor-model-parallel-size 2 --save {root}/ck --save-interval 1"
    if mode == "resume":
        extra += f" --load {root}/ck"
    a = _hy_train_args(world, extra)
    a.global_batch_size = a.current_global_batch_size = 1
    a.num_micro_batches = 1
    t = Trainer(a)
    start = a.iteration
    for it in range(start, 2):
        if mode == "first" and it == 1:
            break
        a.train_iters = it + 1
        t.train(make_hunyuan_forward_step(timestep_generator=torch.Generator().manual_seed(50 + it)))
    shards = sorted(os.listdir(f"{root}/ck/iter_0000001")) if os.path.isdir(f"{root}/ck/iter_0000001") else []
    return start, a.iteration, t.buffer.params.float().clone(), shards


def test_hunyuan_tp2_checkpoint_resumes_exactly(tmp_path):
    full = run_distributed(_hy_tp_resume_worker, 2, str(tmp_path / "full"), "full", timeout=240)
    first = run_distributed(_hy_tp_resume_worker, 2, str(tmp_path / "run"), "first", timeout=240)
    assert [o[:2] for o in first] == [(0, 1), (0, 1)] and first[0][3] == ["mp_rank_00", "mp_rank_01"]
    resumed = run_distributed(_hy_tp_resume_worker, 2, str(tmp_path / "run"), "resume", timeout=240)
    assert [o[:2] for o in resumed] == [(1, 2), (1, 2)]
    for r in range(2):
        assert torch.allclose(resumed[r][2], full[r][2], atol=1e-6)       # each TP rank's shard


def _tp_norm_worker(rank, world):
    from teletron_b200.parallel.tp import tp_shard_dims
    from teletron_b200.train import Trainer, make_hunyuan_forward_step

    t = Trainer(_hy_train_args(world, "--tensor-model-parallel-size 2 --clip-grad 0.05"))
    inner = t.model.module if hasattr(t.model, "module") else t.model
    sharded = set(tp_shard_dims(inner))          # state-dict names: fused projections listed per projection
    gen = torch.Generator().manual_seed(4)
    fwd = make_hunyuan_forward_step(timestep_generator=gen)
    norms = []
    for _ in range(3):
        _, _, gnorm, _ = t.train_step(fwd)
        norms.append(float(gnorm))
    sd = {k: v.detach().float().clone() for k, v in inner.state_dict().items()}
    return norms, {k: v for k, v in sd.items() if k not in sharded}, {k: v for k, v in sd.items() if k in sharded}


def test_tensor_parallel_ranks_share_one_gradient_norm_and_keep_replicated_parameters_identical():
    """Sharded layers start from different slices of one full weight on each tensor-parallel rank, the squared norm
    of sharded parameters is summed over the group and that of replicated ones counted once: every rank clips with
    the same coefficient, so replicated parameters stay bit-identical through clipped steps."""
    (n0, rep0, sh0), (n1, rep1, sh1) = run_distributed(_tp_norm_worker, 2)
    assert n0 == n1 and all(x > 0.05 for x in n0)                        # clipping was active on every step
    assert rep0.keys() == rep1.keys() and len(rep0) > 10
    for k in rep0:
        assert torch.equal(rep0[k], rep1[k]), k
    differing = [k for k in sh0 if k.endswith("weight") and not torch.equal(sh0[k], sh1[k])]
    assert len(differing) == len([k for k in sh0 if k.endswith("weight")])   # no duplicated weight blocks


def test_sharded_layers_initialise_like_the_full_layer():
    from teletron_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear, TPContext

    for cls, dim in ((ColumnParallelLinear, 0), (RowParallelLinear, 1)):
        shards = []
        for r in range(2):
            torch.manual_seed(3)
            shards.append(cls(64, 96, TPContext(None, 2, r), bias=False).weight.detach())
        torch.manual_seed(3)
        full = torch.nn.Linear(64, 96, bias=False).weight.detach()
        assert torch.equal(torch.cat(shards, dim=dim), full)             # same stream, full-layer fan-in
        assert not torch.equal(shards[0], shards[1])
