"""CPU tests of the training stack: flow-matching scheduler vs the reference, LR/WD schedule,
samplers, arguments, recompute policy (recompute count like the reference's block test),
checkpoint save / resume in the Megatron layout, and an end-to-end Trainer run with resume."""
import importlib.util
import os
from argparse import Namespace

import pytest
import torch

from conftest import reference_file
from teletron_b200.data import PretrainingRandomSampler, PretrainingSampler
from teletron_b200.models import FlowMatchScheduler
from teletron_b200.parallel import recompute as rc
from teletron_b200.train import checkpoint as ckpt
from teletron_b200.train import make_forward_step, parse_args
from teletron_b200.train.schedule import OptimizerParamScheduler


def test_flow_match_matches_reference():
    path = reference_file("teletron/models/flow_match.py")
    if path is None:
        pytest.skip("reference tree not available")
    spec = importlib.util.spec_from_file_location("ref_fm", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for kw in (dict(shift=5, sigma_min=0.0, extra_one_step=True), dict(shift=3.0), dict(inverse_timesteps=True)):
        a, b = FlowMatchScheduler(**kw), ref.FlowMatchScheduler(**kw)
        a.set_timesteps(1000, training=True)
        b.set_timesteps(1000, training=True)
        assert torch.allclose(a.sigmas, b.sigmas) and torch.allclose(a.timesteps, b.timesteps)
        assert torch.allclose(a.linear_timesteps_weights, b.linear_timesteps_weights)
        x, n, v = torch.randn(2, 4), torch.randn(2, 4), torch.randn(2, 4)
        t = a.timesteps[417]
        assert torch.allclose(a.add_noise(x, n, t), b.add_noise(x, n, t))
        assert torch.allclose(a.step(v, t, x), b.step(v, t, x))
        assert torch.allclose(a.training_weight(t), b.training_weight(t))
        assert torch.equal(a.training_target(x, n, t), b.training_target(x, n, t))


def test_lr_wd_schedule():
    opt = Namespace(param_groups=[dict(lr=0.0, weight_decay=0.0)])
    s = OptimizerParamScheduler(opt, init_lr=0.0, max_lr=1.0, min_lr=0.1, lr_warmup_steps=10, lr_decay_steps=110,
                                lr_decay_style="cosine", start_wd=0.0, end_wd=0.2, wd_incr_steps=100,
                                wd_incr_style="linear")
    s.step(5)
    assert abs(opt.param_groups[0]["lr"] - 0.5) < 1e-9 and abs(opt.param_groups[0]["weight_decay"] - 0.01) < 1e-9
    s.step(55)  # 60: halfway through the cosine
    assert abs(opt.param_groups[0]["lr"] - 0.55) < 1e-9
    s.step(1000)
    assert opt.param_groups[0]["lr"] == 0.1 and opt.param_groups[0]["weight_decay"] == 0.2
    sd = s.state_dict()
    s2 = OptimizerParamScheduler(opt, 0.0, 1.0, 0.1, 10, 110, "cosine", 0.0, 0.2, 100, "linear")
    s2.load_state_dict({"start_lr": sd["max_lr"], "warmup_iter": 10, "end_iter": 110, "decay_style": "cosine",
                        "num_iters": sd["num_steps"], "min_lr": 0.1})
    assert s2.num_steps == sd["num_steps"]


def test_samplers_resume_and_shard():
    full = [b for b in PretrainingSampler(20, 0, 2, 1, 2)]
    assert full[0] == [2, 3] and full[1] == [6, 7] and len(full) == 5
    resumed = [b for b in PretrainingSampler(20, 8, 2, 1, 2)]
    assert resumed == full[2:]
    a = [b for b in PretrainingRandomSampler(32, 0, 2, 0, 2, seed=7)]
    b = [b for b in PretrainingRandomSampler(32, 0, 2, 1, 2, seed=7)]
    assert not set(sum(a, [])) & set(sum(b, []))          # data sharding: disjoint buckets
    again = [x for x in PretrainingRandomSampler(32, 8, 2, 0, 2, seed=7)]
    assert again == a[2:]                                  # resumable in the middle of an epoch


def test_arguments_surface_and_derivations(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "5")
    monkeypatch.setenv("RANK", "0")
    argv = ("--num-layers 20 --hidden-size 5120 --num-attention-heads 40 --seq-length 512 --max-position-embeddings 4096 "
            "--tokenizer-type NullTokenizer --vocab-size 0 --model ParallelWanModel --task-type wan_i2v_prone "
            "--micro-batch-size 1 --train-iters 10000 --weight-decay 1e-2 --init-method-std 0.006 --clip-grad 0.0 --bf16 "
            "--lr 1e-5 --lr-decay-style constant --lr-warmup-fraction 0 --recompute-granularity full --recompute-method block "
            "--activation-offload --use-distributed-optimizer --recompute-num-layers 40 --no-rope-fusion "
            "--distributed-timeout-minutes 60 --tensor-model-parallel-size 1 --context-parallel-size 2 --distributed-vae "
            "--distributed-vae-world-size 1 --consumer-models-num 1 --dataset-type FakeDataset --split 949,50,1 "
            "--dataloader-type single --num-workers 1 --num-frames 9 --tensorboard-queue-size 10 --log-interval 1 "
            "--save-interval 10000 --eval-interval 10000 --eval-iters 10000").split()

    def extra(p):
        p.add_argument("--moe-step-factor-list", type=float, action="append")
        return p

    a = parse_args(extra, argv + ["--moe-step-factor-list", "0.0", "--moe-step-factor-list", "1.0"])
    assert a.dit_world_size == 4 and a.data_parallel_size == 2 and a.global_batch_size == 2
    assert a.task_type == "i2v" and a.recompute_method == "block" and a.moe_step_factor_list == [0.0, 1.0]
    with pytest.raises(ValueError):
        parse_args(None, ["--context-parallel-size", "3"])


class _CountingLinear(torch.nn.Module):
    calls = 0

    def __init__(self):
        super().__init__()
        self.lin = torch.nn.Linear(32, 32)

    def forward(self, x):
        _CountingLinear.calls += 1
        return torch.tanh(self.lin(x))


@pytest.mark.parametrize("method,k,expect_extra", [("block", 2, 2), ("block", 9, 4), ("uniform", 2, 4), ("uniform", 3, 4)])
def test_recompute_policy_counts_and_grads(method, k, expect_extra):
    torch.manual_seed(0)
    blocks = torch.nn.ModuleList([_CountingLinear() for _ in range(4)])
    x = torch.randn(3, 32, requires_grad=True)
    cfg = Namespace(recompute_granularity=None, recompute_method=method, recompute_num_layers=k, activation_offload=False)
    y0 = rc.run_blocks(blocks, x, (), cfg, True)
    g0 = torch.autograd.grad(y0.sum(), [x] + list(blocks.parameters()))
    cfg.recompute_granularity = "full"
    _CountingLinear.calls = 0
    y1 = rc.run_blocks(blocks, x, (), cfg, True)
    assert torch.equal(y0, y1)
    g1 = torch.autograd.grad(y1.sum(), [x] + list(blocks.parameters()))
    assert _CountingLinear.calls == 4 + expect_extra      # layers + recomputed layers
    for a, b in zip(g0, g1):
        assert torch.allclose(a, b, atol=1e-6)
    _CountingLinear.calls = 0
    rc.run_blocks(blocks, x, (), cfg, False)                 # evaluation: no checkpointing
    assert _CountingLinear.calls == 4


class _PhaseRecorder(torch.nn.Module):
    seen = []

    def __init__(self):
        super().__init__()
        self.lin = torch.nn.Linear(8, 8)

    def forward(self, x):
        _PhaseRecorder.seen.append(rc.forward_is_discarded())
        return self.lin(x)


def test_recompute_marks_the_forward_pass_whose_activations_are_dropped():
    blocks = torch.nn.ModuleList([_PhaseRecorder() for _ in range(3)])
    x = torch.randn(2, 8, requires_grad=True)
    cfg = Namespace(recompute_granularity="full", recompute_method="block", recompute_num_layers=2,
                    activation_offload=False)
    _PhaseRecorder.seen = []
    y = rc.run_blocks(blocks, x, (), cfg, True)
    assert _PhaseRecorder.seen == [True, True, False]       # two checkpointed blocks, one plain
    y.sum().backward()
    assert _PhaseRecorder.seen[3:] == [False, False]         # their recompute passes keep what they save
    assert not rc.forward_is_discarded()


def test_batch_size_rampup_schedule():
    from teletron_b200.train.microbatches import BatchSchedule

    const = BatchSchedule(16, 2, 4)
    assert (const.num_micro_batches, const.current_global_batch_size) == (2, 16)
    assert const.update(10 ** 9) == 2
    # 8 -> 32 in steps of 8 over 240 samples: three increments, 80 samples per level
    ramp = BatchSchedule(32, 2, 4, rampup=["8", "8", "240"])
    seen = [(c, ramp.global_batch_at(c)) for c in (0, 79, 80, 159, 160, 239, 240, 241, 10_000)]
    assert seen == [(0, 8), (79, 8), (80, 16), (159, 16), (160, 24), (239, 24), (240, 32), (241, 32), (10_000, 32)]
    assert ramp.update(160) == 3 and ramp.current_global_batch_size == 24
    odd = BatchSchedule(32, 2, 4, rampup=[4, 4, 70])         # level 4 does not split into passes of 8 samples
    assert odd.update(0, strict=False) == 0
    with pytest.raises(ValueError):
        odd.update(0, strict=True)
    for bad in ([8, 8], [8, 5, 100], [64, 8, 100], [0, 8, 100]):
        with pytest.raises(ValueError):
            BatchSchedule(32, 2, 4, rampup=bad)


def test_trainer_ramps_the_global_batch_and_checkpoints_at_each_level(tmp_path):
    from teletron_b200.train import Trainer
    from teletron_b200.train.checkpoint import read_tracker

    a = _trainer_args(tmp_path, "--rampup-batch-size 1 1 3")   # global batch 1 for the first 3 samples, then 2
    a.train_iters, a.save_interval = 5, 1000
    t = Trainer(a)
    levels = []
    orig = t.train_step

    def spy(fwd, it=None):
        levels.append((a.num_micro_batches, a.current_global_batch_size))
        return orig(fwd, it)

    t.train_step = spy
    t.train(make_forward_step())
    assert levels == [(1, 1), (1, 1), (1, 1), (2, 2), (2, 2)]
    assert a.consumed_train_samples == 1 + 1 + 1 + 2 + 2
    assert read_tracker(str(tmp_path)) == (3, False)            # saved when the level changed, before step 4


def test_trainer_exits_on_sigterm_between_steps_and_saves(tmp_path):
    import signal

    from teletron_b200.train import Trainer
    from teletron_b200.train.checkpoint import read_tracker

    a = _trainer_args(tmp_path, "--exit-signal-handler")
    a.train_iters, a.save_interval = 50, 1000
    t = Trainer(a)
    try:
        orig, calls = t.train_step, []

        def step(fwd, it=None):
            calls.append(1)
            if len(calls) == 2:
                os.kill(os.getpid(), signal.SIGTERM)     # arrives in the middle of step 2
            return orig(fwd, it)

        t.train_step = step
        assert t.train(make_forward_step()) == 2           # step 2 completes, then the loop leaves
        assert read_tracker(str(tmp_path)) == (2, False)
    finally:
        signal.signal(signal.SIGTERM, t._prev_sigterm)


def test_trainer_nan_check_raises(tmp_path):
    from teletron_b200.train import Trainer

    a = _trainer_args(tmp_path, "--check-for-nan-in-loss-and-grad")
    t = Trainer(a)
    fwd = make_forward_step()

    def poisoned(it, model):
        loss, loss_func = fwd(it, model)
        return loss * float("nan"), loss_func

    t.train_step(fwd)                                      # a healthy step passes
    with pytest.raises(RuntimeError, match="non-finite"):
        t.train_step(poisoned)


def _trainer_args(tmp, extra=""):
    argv = (f"--model ParallelWanModel --model-preset wan-tiny --train-iters 4 --micro-batch-size 1 --global-batch-size 2 "
            f"--lr 1e-3 --synthetic-latents --num-frames 5 --video-resolution 64 64 --log-interval 100 --clip-grad 1.0 "
            f"--save {tmp} --save-interval 2 --seed 11 {extra}").split()
    a = parse_args(argv=argv)
    a.text_dim, a.text_len = 64, 16
    return a


def test_trainer_checkpoint_layout_and_exact_resume(tmp_path):
    from teletron_b200.train import Trainer

    gen = torch.Generator().manual_seed(3)
    t1 = Trainer(_trainer_args(tmp_path))
    t1.pretrain(make_forward_step(timestep_generator=gen))
    ref_params = t1.buffer.params.clone()
    root = str(tmp_path)
    assert open(os.path.join(root, "latest_checkpointed_iteration.txt")).read().strip() == "4"
    f2 = os.path.join(root, "iter_0000002", "mp_rank_00", "model_optim_rng.pt")
    assert os.path.exists(f2)
    sd = torch.load(f2, weights_only=False)
    assert sd["checkpoint_version"] == 3.0 and sd["iteration"] == 2
    for key in ("args", "model", "optimizer", "opt_param_scheduler", "rng_state", "num_floating_point_operations_so_far"):
        assert key in sd, key
    assert "blocks.0.self_attn.q.weight" in sd["model"] and sd["args"].consumed_train_samples == 4
    # resume from iteration 2 with the same timestep stream -> identical final parameters
    gen2 = torch.Generator().manual_seed(3)
    for _ in range(2 * 2):
        torch.randint(0, 1000, (1,), generator=gen2)       # the draws of the first two iterations
    a = _trainer_args(tmp_path / "second", f"--load {root} --ckpt-step 2")
    t2 = Trainer(a)
    assert a.iteration == 2 and a.consumed_train_samples == 4
    t2.pretrain(make_forward_step(timestep_generator=gen2))
    assert torch.allclose(t2.buffer.params, ref_params, atol=1e-6)
    # corrupted file -> clear error
    with open(f2, "wb") as fh:
        fh.write(b"truncated")
    with pytest.raises(RuntimeError):
        Trainer(_trainer_args(tmp_path / "third", f"--load {root} --ckpt-step 2"))


def test_phase_timers_are_reported_per_iteration(tmp_path, capsys):
    from teletron_b200.train import Trainer

    a = _trainer_args(tmp_path, "--timing-log-level 2")
    a.train_iters, a.log_interval, a.save_interval = 2, 2, 1000
    t = Trainer(a)
    t.train(make_forward_step())
    got = t.logger.last_timings
    assert set(got) == {"forward-backward", "forward-compute", "backward-compute", "grads-reduce", "optimizer"}
    assert all(v > 0 for v in got.values())
    assert got["forward-backward"] >= 0.9 * (got["forward-compute"] + got["backward-compute"])
    assert "time (ms) | backward-compute:" in capsys.readouterr().out


def test_flags_from_a_yaml_file_with_command_line_override(tmp_path):
    cfg = tmp_path / "run.yaml"
    cfg.write_text("""
model:
  model-preset: wan-tiny
  num_layers: 3
training:
  lr: 3.0e-4
  bf16: true
  train-iters: 7
  no-manual-gc-eval: true
  recompute-granularity: full
seed: 99
""")
    a = parse_args(argv=["--yaml-cfg", str(cfg), "--lr", "1e-5"])
    assert (a.model_preset, a.num_layers, a.train_iters, a.seed, a.bf16) == ("wan-tiny", 3, 7, 99, True)
    assert a.lr == 1e-5                                   # the command line wins over the file
    assert a.manual_gc_eval is False and a.recompute_granularity == "full" and a.recompute_method == "block"
    bad = tmp_path / "bad.yaml"
    bad.write_text("learning-rate: 1.0\n")
    with pytest.raises(ValueError, match="unknown option"):
        parse_args(argv=["--yaml-cfg", str(bad)])
    bad.write_text("recompute-granularity: sometimes\n")
    with pytest.raises(ValueError, match="not one of"):
        parse_args(argv=["--yaml-cfg", str(bad)])


def test_validation_runs_at_the_interval_and_reports_perplexity(tmp_path, capsys):
    import math

    from teletron_b200.train import Trainer

    a = _trainer_args(tmp_path, "--eval-iters 2 --eval-interval 1")
    a.train_iters, a.save_interval = 2, 1000
    t = Trainer(a)
    assert t.valid_data_iterator is not None
    t.pretrain(make_forward_step())
    out = capsys.readouterr().out
    assert "validation loss at iteration 1 |" in out and "validation loss at iteration 2 |" in out
    assert "validation loss at the end of training (iteration 2)" in out
    line = [l for l in out.splitlines() if "validation loss at iteration 1" in l][0]
    val = float(line.split("loss value: ")[1].split(" |")[0])
    ppl = float(line.split("loss PPL: ")[1].split(" |")[0])
    assert abs(ppl - math.exp(min(20.0, val))) < 1e-3 * ppl
    assert a.consumed_valid_samples == 3 * 2 * a.global_batch_size


def test_num_zeros_in_grad_is_counted_on_the_reduced_gradient(tmp_path, capsys):
    from teletron_b200.train import Trainer

    a = _trainer_args(tmp_path, "--log-num-zeros-in-grad --log-interval 1 --log-batch-size-to-tensorboard "
                                "--no-log-loss-scale-to-tensorboard --wandb-project x")
    t = Trainer(a)
    _, _, _, nz = t.train_step(make_forward_step())
    assert nz is not None and 0 <= float(nz) < t.buffer.grads.numel()
    t.optimizer.zero_grad()
    t.buffer.grads.zero_()
    t.optimizer._shard_grads = [t.buffer.grads[s:e] for s, e, _ in t.optimizer.shards]
    assert float(t.optimizer._count_zeros(t.optimizer._shard_grads)) == t.buffer.grads.numel()
    a.train_iters = 1
    t.train(make_forward_step())
    assert "num zeros:" in capsys.readouterr().out


def test_scalar_writer_mirrors_to_a_wandb_run(tmp_path, monkeypatch):
    import sys
    import types

    from teletron_b200.train.telelog import TrainLogger

    logged, inits = [], []

    class Run:
        def log(self, d, step):
            logged.append((d, step))

        def finish(self):
            logged.append("finished")

    fake = types.SimpleNamespace(init=lambda **kw: (inits.append(kw), Run())[1])
    monkeypatch.setitem(sys.modules, "wandb", fake)
    a = _trainer_args(tmp_path, "--wandb-project proj --wandb-exp-name run7")
    w = TrainLogger.make_writer(a)
    assert inits and inits[0]["project"] == "proj" and inits[0]["name"] == "run7" and "lr" in inits[0]["config"]
    w.add_scalar("loss", 0.5, 3)
    w.close()
    assert logged == [({"loss": 0.5}, 3), "finished"]
    a.rank = 0
    a.world_size = 2
    assert TrainLogger.make_writer(a) is None                  # only the last rank writes


def test_training_helpers(capsys):
    from teletron_b200 import train as T
    from teletron_b200.models import wan_config

    lin = torch.nn.Linear(3, 2)
    with torch.no_grad():
        lin.weight.fill_(2.0)
        lin.bias.fill_(1.0)
    wrapped = Namespace(module=Namespace(module=lin))
    assert T.get_attr_wrapped_model(wrapped, "in_features") == 3 and T.get_attr_wrapped_model(wrapped, "nope") is None
    with pytest.raises(AttributeError):
        T.get_attr_wrapped_model(wrapped, "nope", allow_none=False)
    assert abs(T.calc_params_l2_norm(lin) - (6 * 4 + 2) ** 0.5) < 1e-9
    lin(torch.ones(1, 3)).sum().backward()
    assert abs(T.get_grad_norm(lin) - (6 + 2) ** 0.5) < 1e-9
    a = Namespace(train_samples=None, train_iters=10, global_batch_size=4, eval_interval=5, eval_iters=2)
    assert T.get_train_valid_test_num_samples(a) == (40, 3 * 2 * 4, 2 * 4)
    # sample-based training with a ramp 2 -> 6 in steps of 2 over 12 samples (6 per level): batches 2,2,2,4,4,6 reach
    # 20 > 12, then (50 - 20) // 6 = 5 full batches
    r = Namespace(train_iters=None, train_samples=50, global_batch_size=6, micro_batch_size=1, data_parallel_size=2,
                  rampup_batch_size=[2, 2, 12])
    assert T.update_train_iters(r) == 6 + 5 and r.train_iters == 11
    c = Namespace(train_iters=None, train_samples=50, global_batch_size=6, rampup_batch_size=None)
    assert T.update_train_iters(c) == 8
    assert T.is_last_rank()
    T.print_rank_0("zero")
    T.print_rank_last("last")
    T.print_datetime("after setup")
    out = capsys.readouterr().out
    assert "zero" in out and "last" in out and "[after setup] datetime:" in out
    gb = T.report_theoretical_memory(Namespace(data_parallel_size=4, context_parallel_size=2,
                                               use_distributed_optimizer=True), int(1e9))
    assert abs(gb - 1e9 * (2 + 4 + 12 / 8) / 2 ** 30) < 1e-6
    cfg = wan_config("wan2.1-1.3b-t2v")
    assert T.num_floating_point_operations(cfg, 32760, 8) == 8 * T.num_floating_point_operations(cfg, 32760, 1)


def test_exit_interval_and_exit_duration_save_and_leave(tmp_path):
    from teletron_b200.train import Trainer
    from teletron_b200.train.checkpoint import read_tracker

    a = _trainer_args(tmp_path / "a", "--exit-interval 2")
    a.train_iters, a.save_interval = 10, 1000
    assert Trainer(a).train(make_forward_step()) == 2
    assert read_tracker(str(tmp_path / "a")) == (2, False)
    b = _trainer_args(tmp_path / "b", "--exit-duration-in-mins 1")
    b.train_iters, b.save_interval = 10, 1000
    t = Trainer(b)
    t.start_time -= 120.0                                   # the run "started" two minutes ago
    assert t.train(make_forward_step()) == 1
    assert read_tracker(str(tmp_path / "b")) == (1, False)


def test_sample_based_training_uses_sample_denominated_schedules(tmp_path):
    """--train-samples with --lr-warmup-samples / --lr-decay-samples: warm-up ends after 2 samples (= 1 step of 2),
    the cosine reaches --min-lr at 8 samples, weight decay ramps linearly over the run."""
    import math

    from teletron_b200.train import Trainer

    argv = ("--model ParallelWanModel --model-preset wan-tiny --train-samples 8 --micro-batch-size 1 --global-batch-size 2 "
            "--lr 1e-3 --min-lr 1e-4 --lr-decay-style cosine --lr-warmup-samples 2 --lr-decay-samples 8 "
            "--synthetic-latents --num-frames 5 --video-resolution 64 64 --log-interval 100 --seed 11 "
            "--start-weight-decay 0.0 --end-weight-decay 0.1 --weight-decay-incr-style linear").split()
    a = parse_args(argv=argv)
    a.text_dim, a.text_len = 64, 16
    assert a.train_iters == 4 and a.sample_based_training
    t = Trainer(a)
    seen = []
    orig = t.train_step

    def spy(f, it=None):
        r = orig(f, it)
        g = t.optimizer.param_groups[0]
        seen.append((g["lr"], g["weight_decay"]))
        return r

    t.train_step = spy
    t.train(make_forward_step())
    want_lr = [1e-3] + [1e-4 + 0.9e-3 * 0.5 * (1 + math.cos(math.pi * (c - 2) / 6)) for c in (4, 6, 8)]
    assert all(abs(l - w) < 1e-9 for (l, _), w in zip(seen, want_lr)), (seen, want_lr)
    assert all(abs(wd - w) < 1e-9 for (_, wd), w in zip(seen, (0.025, 0.05, 0.075, 0.1)))


def test_load_options_finetune_no_optim_no_rng(tmp_path):
    from teletron_b200.train import Trainer

    first = Trainer(_trainer_args(tmp_path))
    first.pretrain(make_forward_step())                                  # 4 iterations, checkpoints at 2 and 4
    root = str(tmp_path)
    trained = first.buffer.params.clone()
    m_state = first.optimizer.exp_avg[0].clone()
    assert float(m_state.abs().sum()) > 0

    a = _trainer_args(tmp_path / "ft", f"--load {root} --finetune")
    t = Trainer(a)
    assert a.iteration == 0 and a.consumed_train_samples == 0            # weights only: counters start over
    assert torch.equal(t.buffer.params, trained) and float(t.optimizer.exp_avg[0].abs().sum()) == 0
    assert torch.equal(t.optimizer.master[0][:16], trained[:16].float())  # master weights follow the loaded ones

    b = _trainer_args(tmp_path / "noopt", f"--load {root} --no-load-optim --no-load-rng")
    t2 = Trainer(b)
    assert b.iteration == 4 and torch.equal(t2.buffer.params, trained)
    assert float(t2.optimizer.exp_avg[0].abs().sum()) == 0               # optimizer state not restored

    c = _trainer_args(tmp_path / "full", f"--load {root}")
    t3 = Trainer(c)
    assert c.iteration == 4 and torch.equal(t3.optimizer.exp_avg[0], m_state)


def test_sgd_optimizer_matches_torch_sgd():
    from teletron_b200.parallel.ddp import DistributedOptimizer, ParamBuffer

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    ref.load_state_dict(net.state_dict())
    buf = ParamBuffer(net)
    opt = DistributedOptimizer(buf, None, lr=0.1, weight_decay=0.0, kind="sgd", momentum=0.9)
    topt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    for step in range(3):
        x = torch.randn(5, 8)
        opt.zero_grad()
        topt.zero_grad()
        net(x).square().mean().backward()
        ref(x).square().mean().backward()
        opt.step()
        topt.step()
    for (n, p), (_, q) in zip(net.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n


def test_flags_without_effect_are_reported_and_lora_raises(capsys):
    import pytest

    from teletron_b200.train import parse_args

    a = parse_args(argv="--overlap-param-gather --no-rope-fusion --sequence-parallel --no-delay-grad-reduce".split())
    out = capsys.readouterr().out
    assert len(a.inert_flag_notes) == 4 and out.count("NOTE:") == 4
    assert parse_args(argv=[]).inert_flag_notes == []
    with pytest.raises(NotImplementedError):
        parse_args(argv="--lora-rank 8".split())


def test_expert_and_embedding_groups_partition_the_data_parallel_ranks():
    from teletron_b200.parallel.state import Topology

    t = Topology(16, tp=2, cp=2, ep=2)
    assert t.dp == 4
    for groups in (t.ep_groups(), t.dp_modulo_ep_groups()):
        assert sorted(r for g in groups for r in g) == list(range(16)) and all(len(g) == 2 for g in groups)
    assert [0, 4] in t.ep_groups() and [0, 8] in t.dp_modulo_ep_groups() and [0, 1, 4, 5] in t.tp_ep_groups()
    assert all(len(g) == 1 for g in t.embedding_groups())          # one pipeline stage: the rank itself
    p = Topology(8, pp=2)
    assert [0, 4] in p.embedding_groups() and [0] in p.position_embedding_groups()
    import pytest
    with pytest.raises(ValueError):
        Topology(8, ep=3)


def test_memory_snapshot_and_profile_window_drive_their_backends(tmp_path, monkeypatch):
    """MEMORY_SNAPSHOT records and dumps once per step; --profile starts the profiler API, NVTX emission and the
    framework's own ranges at the first profiled step and stops them at the last (fakes stand in for CUDA)."""
    from argparse import Namespace

    from teletron_b200.train import profiling
    from teletron_b200.utils import nvtx

    calls = []

    class FakeMem:
        def _record_memory_history(self, **kw):
            calls.append(("record", kw))

        def _dump_snapshot(self, path):
            calls.append(("dump", path))
            open(path, "w").write("x")

    monkeypatch.setenv("MEMORY_SNAPSHOT", "1")
    monkeypatch.setenv("PROF_SAVE_PATH", str(tmp_path))
    snap = profiling.MemorySnapshot(3, backend=FakeMem())
    snap.begin()
    path = snap.dump(7)
    assert path.endswith("_iter7_rank3.pt") and (tmp_path / path.split("/")[-1]).exists()
    assert [c[0] for c in calls] == ["record", "dump", "record"] and calls[-1][1] == {"enabled": None}
    monkeypatch.delenv("MEMORY_SNAPSHOT")
    assert profiling.MemorySnapshot(0, backend=FakeMem()).dump(1) is None

    events = []

    class FakeRt:
        def cudaProfilerStart(self):
            events.append("start")

        def cudaProfilerStop(self):
            events.append("stop")

    class FakeEmit:
        def __init__(self, **kw):
            events.append("emit")

        def __enter__(self):
            events.append("enter")

        def __exit__(self, *a):
            events.append("exit")

    monkeypatch.setattr(torch.autograd.profiler, "emit_nvtx", FakeEmit)
    monkeypatch.setattr(nvtx, "set_nvtx", lambda on: events.append(("ranges", on)))
    monkeypatch.setattr(profiling, "set_nvtx", nvtx.set_nvtx)
    a = Namespace(profile=True, rank=1, profile_ranks=[1], profile_step_start=2, profile_step_end=4)
    w = profiling.ProfileWindow(a, cudart=FakeRt())
    for it in range(6):
        w.before_step(it)
        w.after_step(it + 1)
    assert events == ["start", "emit", "enter", ("ranges", True), ("ranges", False), "exit", "stop"]
    assert not profiling.ProfileWindow(Namespace(profile=True, rank=0, profile_ranks=[1], profile_step_start=2,
                                                 profile_step_end=4), cudart=FakeRt()).on
    with nvtx.nvtx_range("off-by-default"):
        pass
