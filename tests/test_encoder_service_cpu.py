"""Distributed encoder hand-off on CPU/gloo: wire format, producer -> TP x CP leader -> group
fan-out, identical data across a CP group, resumable sampling, and failure reporting."""
from argparse import Namespace

import pytest
import torch

from dist_utils import run_distributed
from teletron_b200.data import base_encoder as be
from teletron_b200.data.encoder_service import merge_comm_pairs
from teletron_b200.parallel.state import CommPair, Topology


def test_header_round_trip_and_corruption():
    shapes = [(1, 512, 4096), (1, 257, 1280), (1, 20, 21, 60, 104), (1, 16, 21, 60, 104), (1, 16, 21, 60, 104)]
    h = be.encode_header(shapes, seq_no=7, flags=be.FLAG_LAST)
    got, seq, flags = be.decode_header(h)
    assert got == [tuple(s) for s in shapes] and seq == 7 and flags == be.FLAG_LAST
    bad = h.clone(); bad[0] = 123
    with pytest.raises(ValueError):
        be.decode_header(bad)
    bad = h.clone(); bad[3] = 99
    with pytest.raises(ValueError):
        be.decode_header(bad)
    ts = [torch.randn(*s[:2], 8).to(torch.bfloat16) for s in shapes[:2]]
    blob = be.pack_tensors(ts)
    back = be.unpack_tensors(blob, [tuple(t.shape) for t in ts])
    assert all(torch.equal(a, b) for a, b in zip(ts, back))
    with pytest.raises(ValueError):
        be.unpack_tensors(blob[:-1], [tuple(t.shape) for t in ts])


def test_topology_comm_pairs_and_merge():
    topo = Topology(world_size=10, tp=1, cp=2, encoder_ranks=2, replicas=2)  # 8 DiT ranks, 2 replicas of 4
    assert topo.dp == 2 and topo.replica_world == 4
    pairs = topo.comm_pairs()
    assert [p.consumer for p in pairs] == [0, 2, 4, 6]
    assert [p.producer for p in pairs] == [8, 9, 8, 9]
    assert [(p.dp_rank, p.dp_size) for p in pairs] == [(0, 2), (1, 2), (0, 2), (1, 2)]
    merged = merge_comm_pairs([p for p in pairs if p.producer == 8])
    assert merged == [dict(producer=8, dp_rank=0, dp_size=2, consumers=[0, 4])]
    assert topo.coords(5) == dict(replica=1, pp=0, dp=0, cp=1, tp=0)
    assert topo.tp_cp_groups() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert topo.dp_groups(with_cp=True) == [[0, 1, 2, 3], [4, 5, 6, 7]]


def _args(train_iters=3):
    return Namespace(train_iters=train_iters, num_micro_batches=1, micro_batch_size=1, iteration=0,
                     consumed_train_samples=0, consumed_valid_samples=0, video_resolution=[32, 32], num_frames=5,
                     dataset_type="FakeDataset", dataloader_type="single", seed=3, model="ParallelWanModel",
                     encoder_name="synthetic_wan_encoder", task_type="t2v", consumer_models_num=1, text_len=8,
                     text_dim=16, producer_profile=False, moe_step_factor_list=None, distributed_vae=True)


def _service_worker(rank, world, fail):
    import torch.distributed as dist

    try:
        return _service_body(rank, world, fail)
    finally:
        dist.barrier()  # rank 0 hosts the rendezvous store: nobody leaves before everyone is done


def _service_body(rank, world, fail):
    from teletron_b200.data.batch_loader import EncoderTimeout, WanDistBatchLoader
    from teletron_b200.data.encoder_service import producer_process
    from teletron_b200.parallel import state as mpu

    args = _args()
    mpu.initialize_model_parallel(context_parallel_size=2, encoder_world_size=1)  # ranks 0,1 = CP group; 2 = encoder
    if mpu.is_encoder_rank():
        if fail:
            class Broken:
                def setup(self):
                    raise RuntimeError("injected encoder failure")
            with pytest.raises(RuntimeError):
                producer_process(args, encoder=Broken())
            return "failed-as-planned"
        return producer_process(args)
    if fail:
        if rank == 0:  # the TP x CP leader talks to the encoder rank and must see its failure
            with pytest.raises(EncoderTimeout):
                loader = WanDistBatchLoader(args, timeout_s=20.0)
                next(loader)
        return "consumer-saw-failure"
    loader = WanDistBatchLoader(args, timeout_s=20.0)
    sums = []
    for _ in range(args.train_iters):
        b = next(loader)
        assert set(b) == {"context", "latents"} and b["latents"].shape == (1, 16, 2, 4, 4)
        sums.append(float(b["latents"].float().sum()) + float(b["context"].float().sum()))
    return sums


def test_encoder_service_streams_identical_batches_to_cp_group():
    out = run_distributed(_service_worker, 3, False)
    assert out[2] == 3                      # producer issued exactly train_iters samples
    assert out[0] == out[1] and len(set(out[0])) == 3   # same data on both CP ranks, distinct samples


def test_encoder_failure_reaches_the_consumer():
    out = run_distributed(_service_worker, 3, True)
    assert out[2] == "failed-as-planned" and out[0] == "consumer-saw-failure"


def _slow_encoder_body(rank, world):
    """An encoder that takes longer per sample than the consumer: the consumer must never have a receive posted for
    a sample whose sends the producer has not announced (on a GPU such a receive is a kernel that holds an SM while
    it waits), and when the encoder is ahead the next sample is posted before the consumer asks for it."""
    import time

    from teletron_b200.data.batch_loader import WanDistBatchLoader
    from teletron_b200.data.encoder_service import producer_process
    from teletron_b200.models.registry import get_encoder
    from teletron_b200.parallel import state as mpu

    args = _args(train_iters=4)
    mpu.initialize_model_parallel(encoder_world_size=1)      # rank 0 trains, rank 1 encodes
    if mpu.is_encoder_rank():
        enc = get_encoder("synthetic_wan_encoder", device=torch.device("cpu"), args=args)
        inner = enc.encode

        def slow(sample):
            time.sleep(0.4)
            return inner(sample)

        enc.encode = slow
        return producer_process(args, encoder=enc)
    loader = WanDistBatchLoader(args, timeout_s=30.0)
    seen = []
    for i in range(args.train_iters):
        next(loader)
        ahead = loader._pending is not None
        assert loader._posted <= loader._announced()          # nothing posted that is not on its way
        assert loader._posted == loader.received + int(ahead)
        seen.append(ahead)
        if i == 1:
            time.sleep(1.2)                                    # let the encoder get ahead once
    return seen, loader.received


def _slow_encoder_worker(rank, world):
    import torch.distributed as dist

    try:
        return _slow_encoder_body(rank, world)
    finally:
        dist.barrier()


def test_receives_are_posted_only_for_announced_samples():
    out = run_distributed(_slow_encoder_worker, 2, timeout=120)
    seen, received = out[0]
    assert received == 4 and out[1] == 4
    assert seen[0] is False                 # the encoder needs 0.4 s per sample: nothing is on its way right after the first


def test_items_needed_follows_the_batch_size_ramp():
    from argparse import Namespace

    from teletron_b200.data.encoder_service import items_needed

    const = Namespace(train_iters=10, num_micro_batches=3, micro_batch_size=2, rampup_batch_size=None)
    assert items_needed(const, 4) == 6 * 3 * 2
    # dp 2, micro batch 1: global batch 2 for the first 8 samples, then 4 -> per consumer 1, 1, 1, 1, 2, 2
    ramp = Namespace(train_iters=6, num_micro_batches=1, micro_batch_size=1, data_parallel_size=2,
                     global_batch_size=4, rampup_batch_size=["2", "2", "8"])
    assert items_needed(ramp, 0, 0) == 1 + 1 + 1 + 1 + 2 + 2
    assert items_needed(ramp, 4, 8) == 2 + 2                  # resumed after the ramp
