"""Trainer on CPU/gloo ranks: DP + CP with the sharded optimizer, and training fed by an encoder rank."""
import contextlib
import io
import os

import torch

from dist_utils import run_distributed


def _args(world, extra=""):
    from teletron_b200.train import parse_args

    os.environ["WORLD_SIZE"], os.environ["RANK"] = str(world), os.environ.get("RANK", "0")
    argv = (f"--model ParallelWanModel --model-preset wan-tiny --train-iters 2 --micro-batch-size 1 --lr 1e-3 "
            f"--num-frames 5 --video-resolution 64 64 --log-interval 100 --clip-grad 1.0 --seed 5 "
            f"--distributed-backend gloo {extra}").split()

    def extra_args(p):
        p.add_argument("--encoder-name", type=str, default=None)
        p.add_argument("--text-dim", type=int, default=64)
        p.add_argument("--text-len", type=int, default=16)
        return p

    return parse_args(extra_args, argv)


def _dp_cp_worker(rank, world):
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, "--context-parallel-size 2 --use-distributed-optimizer --synthetic-latents --global-batch-size 4")
    assert a.data_parallel_size == 2 and a.num_micro_batches == 2
    t = Trainer(a)
    gen = torch.Generator().manual_seed(9)
    losses = []
    for _ in range(2):
        ld, skipped, gnorm, _ = t.train_step(make_forward_step(timestep_generator=gen))
        losses.append(float(ld["loss"]))
        assert skipped == 0 and torch.isfinite(gnorm)
    return losses, t.buffer.params.clone()


def test_dp2_cp2_sharded_optimizer_keeps_replicas_identical():
    outs = run_distributed(_dp_cp_worker, 4)
    for losses, params in outs[1:]:
        assert torch.equal(params, outs[0][1])           # every rank holds the same parameters after stepping
        assert losses == outs[0][0]                        # the logged loss is the DP mean of CP-summed shares
    assert all(l == l and l > 0 for l in outs[0][0])


def _encoder_fed_worker(rank, world):
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, "--distributed-vae --distributed-vae-world-size 1 --context-parallel-size 2 "
                     "--encoder-name synthetic_wan_encoder --dataset-type FakeDataset --train-iters 5 "
                     "--log-interval 1 --timing-log-level 1")
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    out = io.StringIO()
    with contextlib.redirect_stdout(out):
        t.pretrain(make_forward_step())
    return (float(t.buffer.params.float().abs().sum()), t.train_data_iterator.received, t.train_data_iterator.prefetched,
            out.getvalue().count(" iteration "), bool(t.logger.last_timings))


def test_training_fed_by_an_encoder_rank():
    outs = run_distributed(_encoder_fed_worker, 3, timeout=240)
    assert outs[2] == "encoder-rank-done"
    assert outs[0][0] == outs[1][0] and outs[0][0] > 0
    # the TP x CP leader received all five samples, and for some of them the encoder had promised the sample ahead, so
    # the receive of its payload was posted while the previous sample trained (double buffering)
    assert outs[0][1] == 5 and outs[0][2] >= 1 and outs[1][1:3] == (0, 0)
    # the log lines come from the last rank that trains (the encoder rank behind it never logs), one per iteration,
    # and the timer summary runs over the training ranks only
    assert outs[0][3] == 0 and outs[1][3] == 5 and outs[0][4] and outs[1][4]


def _replica_worker(rank, world):
    """Two timestep-expert replicas of one rank each, fed by one encoder rank (the reference's "consumer models",
    teletron/core/parallel_state.py:192-204): each replica draws its timesteps from its own range, averages
    nothing with the other replica, and the two end up with different weights."""
    from teletron_b200.parallel import state as mpu
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, "--distributed-vae --distributed-vae-world-size 1 --consumer-models-num 2 "
                     "--encoder-name synthetic_wan_encoder --dataset-type FakeDataset --train-iters 3 --log-interval 1")
    a.moe_step_factor_list = [0.0, 0.5, 1.0]
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    assert mpu.get_data_parallel_world_size(with_context_parallel=True) == 1      # replicas are not data-parallel peers
    seen = []
    inner = make_forward_step()

    def fwd(it, model):
        class Tap:
            def __iter__(self_):
                return self_

            def __next__(self_):
                b = next(it)
                seen.append(b.get("timestep_range"))
                return b

        return inner(Tap(), model)

    t.pretrain(fwd)
    return seen, float(t.buffer.params.float().abs().sum()), t.train_data_iterator.received


def test_timestep_expert_replicas_train_apart():
    outs = run_distributed(_replica_worker, 3, timeout=240)
    assert outs[2] == "encoder-rank-done"
    (r0, w0, n0), (r1, w1, n1) = outs[0], outs[1]
    assert r0 == [(0.0, 0.5)] * 3 and r1 == [(0.5, 1.0)] * 3
    assert n0 == 3 and n1 == 3 and w0 != w1 and w0 > 0 and w1 > 0


def _resilience_worker(rank, world, root, mode):
    """mode "full": 3 uninterrupted iterations.  "fail": rank 1 leaves after iteration 1 (between steps, nothing
    of its own in flight); rank 0 finds out at its next collective.  "resume": continue from the last checkpoint."""
    from teletron_b200.train import Trainer, make_forward_step

    extra = ("--use-distributed-optimizer --synthetic-latents --global-batch-size 2 --save-interval 1 "
             f"--save {root}/{'full' if mode == 'full' else 'run'}")
    if mode == "resume":
        extra += f" --load {root}/run"
    a = _args(world, extra)
    a.train_iters = 3
    t = Trainer(a)
    # the timestep stream is a function of the iteration, so a resumed run draws what the first run would have
    def fwd_for(it):
        g = torch.Generator().manual_seed(100 + it)
        return make_forward_step(timestep_generator=g)

    start = a.iteration
    try:
        for it in range(start, a.train_iters):
            if mode == "fail" and rank == 1 and it == 1:
                return "left-after-1"
            a.train_iters = it + 1                 # one iteration per call: train() saves at --save-interval 1
            t.train(fwd_for(it))
    except Exception as e:  # the survivor: its collective fails once the peer is gone
        return f"peer-lost at iteration {a.iteration}: {type(e).__name__}"
    return start, a.iteration, t.buffer.params.float().clone()


def test_a_rank_leaving_is_detected_and_training_resumes_from_the_checkpoint(tmp_path):
    root = str(tmp_path)
    full = run_distributed(_resilience_worker, 2, root, "full", timeout=240)
    assert full[0][:2] == (0, 3) and torch.equal(full[0][2], full[1][2])
    failed = run_distributed(_resilience_worker, 2, root, "fail", timeout=240)
    assert failed[1] == "left-after-1"
    assert isinstance(failed[0], str) and failed[0].startswith("peer-lost at iteration 1"), failed[0]
    from teletron_b200.train.checkpoint import read_tracker

    assert read_tracker(f"{root}/run") == (1, False)              # the last complete checkpoint
    resumed = run_distributed(_resilience_worker, 2, root, "resume", timeout=240)
    assert resumed[0][:2] == (1, 3) and resumed[1][:2] == (1, 3)
    assert torch.equal(resumed[0][2], resumed[1][2])
    assert torch.allclose(resumed[0][2], full[0][2], atol=1e-6)    # same end state as the uninterrupted run


def _ddp_wrapper_worker(rank, world):
    from teletron_b200.parallel.ddp import DistributedDataParallel

    torch.manual_seed(100 + rank)                          # different initial weights: broadcast must equalise them
    net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 2))
    ddp = DistributedDataParallel(net)
    start = ddp.buffer.params.clone()
    g = torch.Generator().manual_seed(7)
    data = torch.randn(world, 2, 4, 6, generator=g)        # [rank, micro-batch, rows, features]
    ddp.zero_grad_buffer()
    with ddp.no_sync():
        ddp(data[rank, 0]).square().mean().backward()
        ddp.start_grad_sync()                              # ignored inside no_sync
        ddp.finish_grad_sync()
        assert all(p.grad is not None for p in net.parameters())
    ddp(data[rank, 1]).square().mean().backward()
    ddp.start_grad_sync()
    ddp.finish_grad_sync()
    assert all(p.grad is None for p in net.parameters())   # folded into the flat buffer
    sd = ddp.state_dict_for_save_checkpoint()
    assert set(sd) == set(net.state_dict())
    return start, ddp.buffer.grads.clone(), data


def test_ddp_wrapper_accumulates_and_averages_like_one_process():
    outs = run_distributed(_ddp_wrapper_worker, 2)
    assert torch.equal(outs[0][0], outs[1][0])              # broadcast_params at construction
    assert torch.equal(outs[0][1], outs[1][1])              # same reduced gradient everywhere
    # one process: same weights, sum over micro-batches, mean over the two ranks' data
    torch.manual_seed(100)
    net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 2))
    data = outs[0][2]
    for r in range(2):
        for mb in range(2):
            (net(data[r, mb]).square().mean() / 2).backward()
    from teletron_b200.parallel.ddp import ParamBuffer

    ref = ParamBuffer(net)
    ref.collect_grads()
    assert torch.allclose(outs[0][1], ref.grads, atol=1e-6)


def _real_clips_worker(rank, world, data_root):
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, "--distributed-vae --distributed-vae-world-size 1 --encoder-name synthetic_wan_encoder "
                     f"--dataset-type VideoFolderDataset --data-path {data_root}")
    a.train_iters = 3                                       # three samples from two clips: the list repeats
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    before = t.buffer.params.float().clone()
    t.pretrain(make_forward_step())
    return a.iteration, float((t.buffer.params.float() - before).abs().sum())


def test_training_on_a_folder_of_clips_through_an_encoder_rank(tmp_path):
    import json

    import numpy as np
    import pytest

    from teletron_b200.utils import video_io

    try:
        import cv2  # noqa: F401
    except ImportError:
        pytest.skip("no video writer backend installed")
    root = tmp_path / "clips"
    root.mkdir()
    rng = np.random.default_rng(0)
    with open(root / "metadata.jsonl", "w") as f:
        for name in ("a.avi", "b.avi"):
            video_io.save_video(list(rng.integers(0, 255, (6, 72, 80, 3), dtype=np.uint8)), str(root / name), fps=8)
            f.write(json.dumps({"video": name, "caption": f"clip {name}"}) + "\n")
    outs = run_distributed(_real_clips_worker, 2, str(root), timeout=240)
    assert outs[1] == "encoder-rank-done"
    assert outs[0][0] == 3 and outs[0][1] > 0


def _per_rank_rng_worker(rank, world, root, mode):
    """Every data-parallel rank draws its own timesteps and noise from its global generators
    (--data-parallel-random-init); a resumed run must continue each rank's stream."""
    from teletron_b200.train import Trainer, make_forward_step

    extra = ("--use-distributed-optimizer --synthetic-latents --global-batch-size 2 --save-interval 1 "
             f"--data-parallel-random-init --num-workers 0 --save {root}/{'full' if mode == 'full' else 'run'}")
    if mode == "resume":
        extra += f" --load {root}/run"
    a = _args(world, extra)
    a.train_iters = 3
    t = Trainer(a)                        # schedules are built for the whole run
    if mode == "first":
        a.train_iters = 1                 # ... of which the first launch only gets through one iteration
    start = a.iteration
    # different on the two ranks, and part of the stream a resume continues (so a resumed run must not draw it again)
    drawn = float(torch.rand(1)) if mode != "resume" else None
    t.train(make_forward_step())
    return start, a.iteration, drawn, t.buffer.params.float().clone()


def test_per_rank_random_streams_survive_a_resume(tmp_path):
    root = str(tmp_path)
    full = run_distributed(_per_rank_rng_worker, 2, root, "full", timeout=240)
    assert full[0][2] != full[1][2]                                       # the ranks really use different streams
    first = run_distributed(_per_rank_rng_worker, 2, root, "first", timeout=240)
    assert [o[:2] for o in first] == [(0, 1), (0, 1)] and first[0][2] == full[0][2] and first[1][2] == full[1][2]
    sd = torch.load(f"{root}/run/iter_0000001/mp_rank_00/model_optim_rng.pt", weights_only=False)
    assert len(sd["rng_state"]) == 2                                      # one state per data-parallel rank
    resumed = run_distributed(_per_rank_rng_worker, 2, root, "resume", timeout=240)
    assert [o[:2] for o in resumed] == [(1, 3), (1, 3)]
    assert torch.allclose(resumed[0][3], full[0][3], atol=1e-6) and torch.equal(resumed[0][3], resumed[1][3])


def _early_exit_worker(rank, world):
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, "--distributed-vae --distributed-vae-world-size 1 --encoder-name synthetic_wan_encoder "
                     "--dataset-type FakeDataset --exit-interval 2")
    a.train_iters = 10                                       # the encoder rank plans for ten samples
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    t.pretrain(make_forward_step())
    it = t.train_data_iterator
    return a.iteration, it.finished, it._pending is None


def test_an_early_exit_stops_the_encoder_rank_and_closes_the_stream():
    """--exit-interval ends training after 2 of 10 iterations: the encoder rank is told to stop, sends what it had in
    flight plus a stop header (which completes the consumer's prefetched receive), and both ranks reach the final
    barrier instead of hanging."""
    outs = run_distributed(_early_exit_worker, 2, timeout=120)
    assert outs[1] == "encoder-rank-done"
    assert outs[0] == (2, True, True)


def _sigterm_job_worker(rank, world, root):
    import signal

    from teletron_b200.data.encoder_service import store
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, "--distributed-vae --distributed-vae-world-size 1 --encoder-name synthetic_wan_encoder "
                     f"--dataset-type FakeDataset --exit-signal-handler --save {root} --save-interval 1000")
    a.train_iters = 10
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    orig, calls = t.train_step, []

    def step(fwd, it=None):
        calls.append(1)
        if len(calls) == 2:                                 # the scheduler's SIGTERM reaches every process of the job
            os.kill(int(store().get("tt_pid_1").decode()), signal.SIGTERM)
            os.kill(os.getpid(), signal.SIGTERM)
        return orig(fwd, it)

    t.train_step = step
    try:
        t.pretrain(make_forward_step())
    finally:
        signal.signal(signal.SIGTERM, t._prev_sigterm)
    return a.iteration


def test_sigterm_to_the_whole_job_saves_and_leaves_with_the_encoder_rank(tmp_path):
    from teletron_b200.train.checkpoint import read_tracker

    outs = run_distributed(_sigterm_job_worker, 2, str(tmp_path), timeout=120)
    assert outs == [2, "encoder-rank-done"]
    assert read_tracker(str(tmp_path)) == (2, False)


def _overlap_worker(rank, world, overlap, sharded):
    from teletron_b200.train import Trainer, make_forward_step

    extra = ("--synthetic-latents --global-batch-size 4 --ddp-bucket-size 20000 "
             + ("--use-distributed-optimizer " if sharded else "")
             + ("--overlap-grad-reduce" if overlap else "--no-overlap-grad-reduce"))
    t = Trainer(_args(world, extra))
    assert t.optimizer.overlap == overlap and len(t.buffer.buckets) > 8
    gen = torch.Generator().manual_seed(9)
    norms, fired = [], []
    for _ in range(2):
        _, _, gnorm, _ = t.train_step(make_forward_step(timestep_generator=gen))
        norms.append(float(gnorm))
        fired.append(t.optimizer.fired_in_backward)
    return norms, fired, t.buffer.params.clone()


def test_bucket_reductions_started_during_backward_change_no_bit():
    """--overlap-grad-reduce starts most buckets' reductions from the gradient-ready hooks of the last micro-batch;
    parameters and gradient norm are bit-identical to the run that reduces after backward (plain and sharded)."""
    for sharded in (False, True):
        plain = run_distributed(_overlap_worker, 2, False, sharded)
        over = run_distributed(_overlap_worker, 2, True, sharded)
        assert plain[0][1] == [0, 0] and min(over[0][1]) > len(over[0][1])      # most buckets fired from the hooks
        for r in range(2):
            assert over[r][0] == plain[r][0]
            assert torch.equal(over[r][2], plain[r][2]) and torch.equal(over[r][2], over[0][2])


def _reshard_worker(rank, world, root, mode):
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, f"--synthetic-latents --global-batch-size 2 --use-distributed-optimizer --ddp-bucket-size "
                     f"{20000 if mode == 'save' else 33000} --save {root} --load {root} --train-iters 3")
    t = Trainer(a)
    if mode == "save":
        gen = torch.Generator().manual_seed(9)
        for _ in range(2):
            t.train_step(make_forward_step(timestep_generator=gen))
        a.iteration = 2
        t.save(2)
        full = t.optimizer.gather_full_state()
        return None if full is None else {k: full[k] for k in ("exp_avg", "exp_avg_sq")} | {"index": full["layout"]["index"]}
    assert a.iteration == 2
    full = t.optimizer.gather_full_state()
    return None if full is None else {k: full[k] for k in ("exp_avg", "exp_avg_sq")} | {"index": full["layout"]["index"]}


def test_sharded_optimizer_state_moves_to_another_dp_size_and_bucket_size(tmp_path):
    """distrib_optim.pt stores the buffer layout, so a run with another data-parallel size (other padding) and
    another bucket size places every parameter's moments where its own layout wants them."""
    saved = run_distributed(_reshard_worker, 2, str(tmp_path), "save")[0]
    loaded = run_distributed(_reshard_worker, 1, str(tmp_path), "load")[0]
    assert saved["index"].keys() == loaded["index"].keys()
    moved = 0
    for k, (o, n) in saved["index"].items():
        lo, ln = loaded["index"][k]
        assert ln == n
        moved += int(lo != o)
        for key in ("exp_avg", "exp_avg_sq"):
            assert torch.equal(saved[key][o:o + n], loaded[key][lo:lo + n]), (k, key)
    assert float(saved["exp_avg_sq"].abs().sum()) > 0


def _dist_ckpt_worker(rank, world, root, mode):
    from teletron_b200.train import Trainer, make_forward_step

    flags = "--use-dist-ckpt --ckpt-fully-parallel-save" if mode != "auto" else "--auto-detect-ckpt-format"
    a = _args(world, f"--synthetic-latents --global-batch-size 2 --use-distributed-optimizer --ddp-bucket-size 20000 "
                     f"--save {root} --load {root} --train-iters 4 {flags}")
    t = Trainer(a)
    gen = torch.Generator().manual_seed(9)
    fwd = make_forward_step(timestep_generator=gen)
    def step():
        t.train_step(fwd)
        a.iteration += 1
        a.consumed_train_samples += a.global_batch_size

    if mode == "save":
        step(), step()
        t.save(2)
        step(), step()
        return t.buffer.params.clone(), torch.cat([m.reshape(-1) for m in t.optimizer.exp_avg]), sorted(os.listdir(
            os.path.join(root, "iter_0000002")))
    assert a.iteration == 2 and t.optimizer.step_count == 2 and a.consumed_train_samples == 4
    for _ in range(2):       # the generator restarts, so replay its first two draws to stay on the saved run's stream
        torch.randint(0, 1000, (1,), generator=gen)
    step(), step()
    return t.buffer.params.clone(), torch.cat([m.reshape(-1) for m in t.optimizer.exp_avg]), []


def test_distributed_checkpoint_resumes_exactly(tmp_path):
    """--use-dist-ckpt: every rank writes its own shares (no gather), replicated tensors once; resuming from the
    directory (named by the flag or detected from metadata.json) continues bit for bit."""
    saved = run_distributed(_dist_ckpt_worker, 2, str(tmp_path), "save")
    files = saved[0][2]
    assert "metadata.json" in files and "common.pt" in files and ".metadata" in files
    assert sum(f.endswith(".distcp") for f in files) == 2 and "mp_rank_00" not in files
    for mode in ("load", "auto"):
        got = run_distributed(_dist_ckpt_worker, 2, str(tmp_path), mode)
        for r in range(2):
            assert torch.equal(got[r][0], saved[r][0]) and torch.equal(got[r][1], saved[r][1])


def _zero2_worker(rank, world, root, mode):
    from teletron_b200.train import Trainer, make_forward_step

    a = _args(world, f"--synthetic-latents --global-batch-size 2 --use-zero2 --context-parallel-size 2 "
                     f"--save {root} --load {root} --train-iters 3")
    t = Trainer(a)
    assert t.optimizer.sharded
    if mode == "save":
        gen = torch.Generator().manual_seed(9)
        t.train_step(make_forward_step(timestep_generator=gen))
        a.iteration = 1
        t.save(1)
        return sorted(os.listdir(os.path.join(root, "iter_0000001", "mp_rank_00"))), [m.clone() for m in t.optimizer.exp_avg_sq]
    assert a.iteration == 1 and t.optimizer.step_count == 1
    return [], [m.clone() for m in t.optimizer.exp_avg_sq]


def test_zero2_flag_writes_one_optimizer_shard_per_rank(tmp_path):
    saved = run_distributed(_zero2_worker, 2, str(tmp_path), "save")
    assert saved[0][0] == ["model_optim_rng.pt", "zero2_optim_dp0_cp0.pt", "zero2_optim_dp0_cp1.pt"]
    loaded = run_distributed(_zero2_worker, 2, str(tmp_path), "load")
    for r in range(2):
        for a_, b_ in zip(saved[r][1], loaded[r][1]):
            assert torch.equal(a_, b_) and float(a_.abs().sum()) > 0
