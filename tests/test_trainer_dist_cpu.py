"""Trainer on CPU/gloo ranks: DP + CP with the sharded optimizer, and training fed by an encoder rank."""
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
                     "--encoder-name synthetic_wan_encoder --dataset-type FakeDataset")
    try:
        t = Trainer(a)
    except SystemExit:
        return "encoder-rank-done"
    t.pretrain(make_forward_step())
    return float(t.buffer.params.float().abs().sum())


def test_training_fed_by_an_encoder_rank():
    outs = run_distributed(_encoder_fed_worker, 3, timeout=240)
    assert outs[2] == "encoder-rank-done"
    assert outs[0] == outs[1] and outs[0] > 0
