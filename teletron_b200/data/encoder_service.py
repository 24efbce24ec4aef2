"""Producer loop of the distributed multimodal encoders: what an encoder rank runs instead of
training (teletron/core/distributed/distributed_encoder.py:59-192).

Each encoder rank serves the TP x CP leaders assigned to it by ``Topology.comm_pairs``:
  1. receive ``int64[3] = (iteration, consumed_train, consumed_valid)`` from every consumer, so
     the data iterators resume where training stopped;
  2. merge consumers that must see identical data (same producer, dp_rank, dp_size — the same
     DP rank in different timestep-expert replicas);
  3. loop: reap completed sends, keep up to ``QUEUE_DEPTH`` encoded samples per consumer
     group, send header then payload with at most one sample in flight per consumer, publish a
     heartbeat in the rendezvous store.
Both sides know how many samples the run needs, so the stream ends without dangling sends; an
early stop is negotiated through the store (``stop`` key, then the producer publishes how many
samples it issued and the consumer drains them).  A failure in the encoder is reported in the
store so consumers raise instead of waiting forever (the reference aborts the world group).
"""
from __future__ import annotations

import collections
import os
import time
import traceback
from typing import Dict, List

import torch
import torch.distributed as dist

from ..models.registry import encoder_for_model, get_encoder
from ..parallel import state as mpu
from ..parallel.state import CommPair
from .base_encoder import FLAG_LAST, FLAG_NEXT_SAME, FLAG_STOP, encode_header, pack_tensors

QUEUE_DEPTH = 2
MAX_OUTSTANDING_SENDS = 1
POLL_SECONDS = 0.002


def store():
    from torch.distributed.distributed_c10d import _get_default_store

    return _get_default_store()


def store_has(key: str) -> bool:
    try:
        return bool(store().check([key]))
    except Exception:
        return False


class PolledWork:
    """Non-blocking completion test for a p2p request on any backend.  NCCL requests answer
    ``is_completed()`` truthfully; gloo send/recv requests only flip it inside ``wait()``, so for
    those a helper thread blocks in ``wait()`` and the caller polls the thread."""

    def __init__(self, work, backend: str):
        self.work = work
        self.error = None
        self.thread = None
        if backend != "nccl":
            import threading

            self.thread = threading.Thread(target=self._block, daemon=True)
            self.thread.start()

    def _block(self):
        try:
            self.work.wait()
        except Exception as e:  # surfaced by done()
            self.error = e

    def done(self) -> bool:
        if self.thread is None:
            return self.work.is_completed()
        if self.thread.is_alive():
            return False
        if self.error is not None:
            raise self.error
        return True


def merge_comm_pairs(pairs: List[CommPair]) -> List[Dict]:
    """Group consumers that share (producer, dp_rank, dp_size): they receive identical samples."""
    groups: Dict[tuple, Dict] = collections.OrderedDict()
    for p in pairs:
        key = (p.producer, p.dp_rank, p.dp_size)
        g = groups.setdefault(key, dict(producer=p.producer, dp_rank=p.dp_rank, dp_size=p.dp_size, consumers=[]))
        g["consumers"].append(p.consumer)
    return list(groups.values())


def items_needed(args, iteration: int, consumed_train_samples: int = 0) -> int:
    """Samples one consumer will request from `iteration` to the end of training.  With
    ``--rampup-batch-size`` the global batch grows with the samples consumed, so the count follows the
    same schedule the trainer steps through."""
    remaining = max((args.train_iters or 0) - iteration, 0)
    if not getattr(args, "rampup_batch_size", None):
        return remaining * args.num_micro_batches * args.micro_batch_size
    from ..train.microbatches import BatchSchedule

    sched = BatchSchedule(args.global_batch_size, args.micro_batch_size, args.data_parallel_size,
                          args.rampup_batch_size)
    consumed, total = int(consumed_train_samples), 0
    for _ in range(remaining):
        n_mb = sched.update(consumed, strict=True)
        total += n_mb * args.micro_batch_size
        consumed += sched.current_global_batch_size
    return total


def _comm_device(backend: str):
    return torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")


def producer_process(args, encoder=None, dataset=None):
    rank = dist.get_rank()
    backend = dist.get_backend()
    dev = _comm_device(backend)
    st = store()
    if getattr(args, "exit_signal_handler", False):
        # a scheduler's SIGTERM reaches every process of the job: the DiT ranks save and then ask this rank to stop,
        # so it has to outlive the signal and keep serving until that request arrives
        import signal

        signal.signal(signal.SIGTERM, lambda signum, frame: print(
            f"[encoder rank {rank}] SIGTERM received: serving until the consumers close their streams", flush=True))
    try:
        st.set(f"tt_pid_{rank}", str(os.getpid()))
        pairs = [p for p in mpu.get_comm_pair() if p.producer == rank]
        if not pairs:
            dist.barrier()
            return 0
        if encoder is None:
            encoder = get_encoder(getattr(args, "encoder_name", None) or encoder_for_model(args.model), device=dev,
                                  args=args)
        encoder.setup()
        # 1. resume counters
        info = torch.zeros((len(pairs), 3), dtype=torch.int64, device=dev)
        for req in [dist.irecv(info[i], src=p.consumer) for i, p in enumerate(pairs)]:
            req.wait()
        iteration, consumed_train = int(info[0, 0]), int(info[0, 1])
        total = items_needed(args, iteration, consumed_train)
        # 2. one data iterator per group of consumers that share data
        groups = merge_comm_pairs(pairs)
        if dataset is None:
            from . import build_dataset

            h, w = args.video_resolution
            dataset = build_dataset(args.dataset_type, num_frames=args.num_frames, height=h, width=w, seed=args.seed,
                                    data_path=getattr(args, "data_path", None),
                                    min_length=consumed_train + total * max(g["dp_size"] for g in groups))
        from .samplers import build_data_loader

        iters = []
        for g in groups:
            dl = build_data_loader(dataset, consumed_train, args.micro_batch_size, g["dp_rank"], g["dp_size"],
                                   args.dataloader_type, 0, args.seed, pin_memory=False,
                                   collate_fn=lambda b: b[0] if len(b) == 1 else b)
            iters.append(iter(dl))
        queues = {p.consumer: collections.deque() for p in pairs}
        issued = {p.consumer: 0 for p in pairs}
        inflight = []  # (work, consumer, keepalive tensors)
        prof = None
        if getattr(args, "producer_profile", False):
            from ..train.profiling import make_torch_profiler

            prof = make_torch_profiler(args, "producer")
            prof.__enter__()
        stopping = False
        encoded, encode_seconds, t_loop = 0, 0.0, time.time()
        promised = {p.consumer: False for p in pairs}   # the last header sent to this consumer carried FLAG_NEXT_SAME

        def send_next(c, may_promise=True):
            shapes, blob = queues[c].popleft()
            flags = FLAG_LAST if issued[c] + 1 >= total else 0
            # promise the following sample when it is already encoded and looks the same: the consumer then
            # receives it into its second buffer while this one trains
            promised[c] = bool(may_promise and not flags and queues[c] and queues[c][0][0] == shapes)
            if promised[c]:
                flags |= FLAG_NEXT_SAME
            hdr = encode_header(shapes, issued[c], flags).to(dev)
            # announced first, then sent: the consumer posts its receives only for announced samples (they never idle
            # on its GPU while a sample is still being encoded), and the first NCCL send to a peer may block until
            # that peer joins with its receive, which it only does once it has seen the announcement
            st.add(f"tt_sent_{rank}_{c}", 1)
            inflight.append((PolledWork(dist.isend(hdr, dst=c), backend), c, hdr))
            inflight.append((PolledWork(dist.isend(blob, dst=c), backend), c, blob))
            issued[c] += 1

        while True:
            st.set(f"tt_hb_{rank}", str(time.time()))
            inflight = [x for x in inflight if not x[0].done()]
            if not stopping and store_has("tt_stop"):
                stopping = True
            done = all(issued[c] >= total for c in issued) or (stopping and not any(promised.values()))
            if done and not inflight:
                break
            if not stopping:
                for g, it in zip(groups, iters):
                    first = g["consumers"][0]
                    if issued[first] + len(queues[first]) < total and len(queues[first]) < QUEUE_DEPTH:
                        t_enc = time.time()
                        tensors, _ = encoder.encode(next(it))
                        blob = pack_tensors(tensors).to(dev)
                        if dev.type == "cuda":
                            # the sample is complete before it is queued (and timed).  Only the encoder's own stream:
                            # a device-wide wait would also wait for sends the consumer has not picked up yet, and
                            # the encoder could never get more than one sample ahead
                            torch.cuda.current_stream().synchronize()
                        encode_seconds += time.time() - t_enc
                        encoded += 1
                        shapes = [tuple(t.shape) for t in tensors]
                        for c in g["consumers"]:
                            queues[c].append((shapes, blob))
            for p in pairs:
                c = p.consumer
                if stopping and not promised[c]:
                    continue                      # after a stop request only promised samples still go out
                if queues[c] and sum(1 for x in inflight if x[1] == c) < MAX_OUTSTANDING_SENDS * 2:
                    send_next(c, may_promise=not stopping)   # a sample sent while stopping promises nothing further
            if prof is not None:
                prof.step()
            time.sleep(POLL_SECONDS)
        if stopping:
            # close every unfinished stream with a payload-less header: the consumer's prefetched header receive
            # completes instead of staying in flight until the process group is torn down
            closing = []
            for c, n in issued.items():
                if n < total:
                    hdr = encode_header([], n, FLAG_STOP).to(dev)
                    st.add(f"tt_sent_{rank}_{c}", 1)
                    closing.append((PolledWork(dist.isend(hdr, dst=c), backend), hdr))
            for c, n in issued.items():
                st.set(f"tt_issued_{rank}_{c}", str(n))
            t_end = time.time() + 60.0
            while any(not w.done() for w, _ in closing) and time.time() < t_end:
                time.sleep(POLL_SECONDS)
        else:
            for c, n in issued.items():
                st.set(f"tt_issued_{rank}_{c}", str(n))
        if prof is not None:
            prof.__exit__(None, None, None)
        if encoded:
            wall = max(time.time() - t_loop, 1e-9)
            print(f"[encoder rank {rank}] encoded {encoded} samples in {wall:.1f} s: {encode_seconds / encoded:.3f} s per "
                  f"sample of encoder time ({encoded / max(encode_seconds, 1e-9):.2f} samples/s when busy), "
                  f"{sum(issued.values())} messages sent", flush=True)
        return sum(issued.values())
    except Exception:
        msg = traceback.format_exc()
        try:
            st.set(f"tt_failed_{rank}", msg[-2000:])
        except Exception:
            pass
        print(f"[encoder rank {rank}] failed:\n{msg}", flush=True)
        raise
