"""Consumer side of the encoder service: the iterator a DiT rank trains from when encoders run
on dedicated ranks (teletron/train/consumer_dataloader.py:18-282).

The TP x CP leader receives (header, payload) from its producer with a watchdog (timed polling
of the receive, producer heartbeat and failure keys in the store, so a dead encoder raises an
error instead of hanging the job) and fans the sample out to its TP x CP group with two broadcasts
(header, flat payload) instead of pickled metadata plus one broadcast per tensor.

Double buffering without idle receive kernels: a receive is posted only once the producer has announced (a
counter in the store, bumped right before it issues the sends) the sample, so an NCCL receive kernel never sits on the GPU waiting
for an encoder that is still encoding (such a kernel holds an SM for as long as it waits, and a persistent GEMM
that counts on every SM then runs at half speed: measured 795 against 680 ms per step).  When the following
sample is already on its way at the end of a receive, its header and, if the header before promised the same
shapes (``FLAG_NEXT_SAME``), its payload are posted at once into a second buffer and cross NVLink while the
current sample trains.  Headers are read on the host through a pinned buffer and a side stream: neither the
receive nor the fan-out waits for the training kernels already queued on the compute stream.
``timestep_range`` is attached for timestep-expert replicas from ``--moe-step-factor-list``.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..parallel import state as mpu
from .base_encoder import (FLAG_LAST, FLAG_NEXT_SAME, FLAG_STOP, HEADER_INTS, decode_header, encode_header, numel_of,
                           unpack_tensors)
from .encoder_service import PolledWork, store, store_has

WAN_SCHEMA = ["context", "clip_feature", "image_emb_y", "latents", "noise"]
HUNYUAN_SCHEMA = ["prompt_embeds", "clip_text_embed", "first_ref_image", "latents"]


class EncoderTimeout(RuntimeError):
    pass


class DistBatchLoader:
    schema: List[str] = WAN_SCHEMA

    def __init__(self, args, timeout_s: float = 600.0, heartbeat_stale_s: float = 120.0):
        self.args = args
        self.timeout_s, self.heartbeat_stale_s = timeout_s, heartbeat_stale_s
        self.backend = dist.get_backend()
        self.dev = (torch.device("cuda", torch.cuda.current_device()) if self.backend == "nccl"
                    else torch.device("cpu"))
        self.rank = dist.get_rank()
        pairs = [p for p in mpu.get_comm_pair() if p.consumer == self.rank]
        self.pair = pairs[0] if pairs else None
        self.is_leader = self.pair is not None
        self.group = mpu.get_tensor_context_parallel_group()
        self.group_size = mpu.get_tensor_context_parallel_world_size()
        self.src = mpu.get_tensor_context_parallel_src_rank()
        self.received = 0
        self.prefetched = 0          # samples whose payload receive was posted before their header arrived
        self.finished = False
        self._pending = None
        self._pending_payload = None
        self._posted = 0             # header receives posted so far (never ahead of the producer's announced sends)
        self._next_numel = None      # payload size of the following sample, when the last header promised it
        self._side = None
        factors = getattr(args, "moe_step_factor_list", None)
        self.timestep_range = None
        if factors and len(factors) >= 2:
            rep = mpu.get_topology().coords(self.rank)["replica"]
            if rep + 1 < len(factors):
                self.timestep_range = (float(factors[rep]), float(factors[rep + 1]))
        if self.is_leader:
            info = torch.tensor([args.iteration, args.consumed_train_samples, args.consumed_valid_samples],
                                dtype=torch.int64, device=self.dev)
            self._wait(dist.isend(info, dst=self.pair.producer), "the resume handshake")

    # ---- host view of a header without touching the compute stream ---------------------------
    def _header_to_host(self, hdr: torch.Tensor):
        if not hdr.is_cuda:
            return hdr
        if self._side is None:
            self._side = torch.cuda.Stream()
            self._hdr_host = torch.empty(HEADER_INTS, dtype=torch.int32).pin_memory()
            self._hdr_event = torch.cuda.Event()
        with torch.cuda.stream(self._side):
            self._hdr_host.copy_(hdr, non_blocking=True)
            self._hdr_event.record(self._side)
        self._hdr_event.synchronize()
        return self._hdr_host.clone()

    # ---- leader-side receive with watchdog ------------------------------------------------
    def _announced(self) -> int:
        """Samples (and stop headers) the producer has announced to this rank: encoded, their sends being issued."""
        return int(store().add(f"tt_sent_{self.pair.producer}_{self.rank}", 0))

    def _post_header(self):
        hdr = torch.zeros(HEADER_INTS, dtype=torch.int32, device=self.dev)
        self._pending = (PolledWork(dist.irecv(hdr, src=self.pair.producer), self.backend), hdr)
        self._posted += 1

    def _prefetch(self):
        """Posts the receives of the following sample if the producer has already announced it."""
        if self._pending is not None or self.finished or self._announced() <= self._posted:
            return
        self._post_header()
        if self._next_numel is not None:
            self._pending_payload = self._post_payload(self._next_numel)

    def _post_payload(self, numel: int):
        blob = torch.empty(numel, dtype=torch.bfloat16, device=self.dev)
        return PolledWork(dist.irecv(blob, src=self.pair.producer), self.backend), blob

    def _wait(self, work, what: str):
        polled = work if isinstance(work, PolledWork) else PolledWork(work, self.backend)
        self._wait_until(polled.done, what)
        if polled.thread is None:
            polled.work.wait()

    def _wait_until(self, ready, what: str):
        t0 = time.time()
        prod = self.pair.producer
        while not ready():
            if store_has(f"tt_failed_{prod}"):
                raise EncoderTimeout(f"encoder rank {prod} reported a failure: "
                                     f"{store().get(f'tt_failed_{prod}').decode(errors='replace')[-500:]}")
            now = time.time()
            if now - t0 > self.timeout_s:
                raise EncoderTimeout(f"timed out after {self.timeout_s:.0f}s waiting for {what} from encoder rank {prod}")
            if store_has(f"tt_hb_{prod}") and now - t0 > 5.0:
                hb = float(store().get(f"tt_hb_{prod}").decode())
                if now - hb > self.heartbeat_stale_s:
                    raise EncoderTimeout(f"encoder rank {prod} stopped sending heartbeats {now - hb:.0f}s ago")
            time.sleep(0.001)

    def _wait_group(self, work, what: str):
        """A follower's wait for a collective of its TP x CP group, on the host and bounded."""
        polled = PolledWork(work, self.backend)
        t0 = time.time()
        while not polled.done():
            if time.time() - t0 > self.timeout_s:
                raise EncoderTimeout(f"timed out after {self.timeout_s:.0f}s waiting for {what} from rank {self.src}")
            time.sleep(0.0005)
        if polled.thread is None:
            polled.work.wait()

    def _receive(self):
        if self._pending is None:
            self._wait_until(lambda: self._announced() > self._posted, "the next sample")
            self._post_header()
        work, hdr = self._pending
        self._wait(work, "a sample header")
        shapes, seq, flags = decode_header(self._header_to_host(hdr))
        if flags & FLAG_STOP:                      # the producer closed the stream after a stop request
            self.finished, self._pending = True, None
            return None
        if seq != (self.received & 0x7FFFFFFF):
            raise ValueError(f"encoder stream out of order: got sample {seq}, expected {self.received}")
        numel = numel_of(shapes)
        if self._pending_payload is not None:      # posted when the previous header promised this sample
            pwork, blob = self._pending_payload
            self._pending_payload = None
            if blob.numel() != numel:
                raise ValueError("encoder stream broke its promise: the sample announced as same-shaped is not")
            self.prefetched += 1
        else:
            pwork, blob = self._post_payload(numel)
        # receives match the producer's sends in order: header n, payload n, header n+1, payload n+1
        self._pending = None
        self._next_numel = numel if (flags & FLAG_NEXT_SAME) else None
        if flags & FLAG_LAST:
            self.finished = True
        self._wait(pwork, "a sample payload")
        self.received += 1
        self._prefetch()                           # the following sample, if it is already on its way
        return hdr, blob, shapes

    # ---- iterator -------------------------------------------------------------------------------
    def __iter__(self):
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        stop = False
        if self.is_leader:
            got = None
            if not self.finished:
                got = self._receive()
            if got is None:
                stop = True
                hdr, blob, shapes = encode_header([], self.received, FLAG_STOP).to(self.dev), None, None
            else:
                hdr, blob, shapes = got
        else:
            hdr = torch.zeros(HEADER_INTS, dtype=torch.int32, device=self.dev)
            blob, shapes = None, None
        if self.group_size > 1:
            # the header always goes round first, a stop header when the stream is over, so that followers leave
            # with the leader instead of waiting in a broadcast that never comes
            if self.is_leader:
                dist.broadcast(hdr, self.src, group=self.group)
            else:
                # the header is read on the host through a side stream, which does not wait for the broadcast by
                # itself: poll the collective's completion first (reading early returned zeros, a "bad magic number")
                self._wait_group(dist.broadcast(hdr, self.src, group=self.group, async_op=True), "the sample header")
                shapes, _, flags = decode_header(self._header_to_host(hdr))
                stop = bool(flags & FLAG_STOP)
                if not stop:
                    blob = torch.empty(numel_of(shapes), dtype=torch.bfloat16, device=self.dev)
            if not stop:
                dist.broadcast(blob, self.src, group=self.group)
        if stop:
            raise StopIteration
        tensors = unpack_tensors(blob, shapes)
        batch = {}
        for name, t in zip(self.schema, tensors):
            if t.numel() > 0:
                batch[name] = t
        if self.timestep_range is not None:
            batch["timestep_range"] = self.timestep_range
        return batch

    def close(self):
        """Early stop: ask producers to stop and drain what they already issued."""
        if not self.is_leader or self.finished:
            return
        st = store()
        st.set("tt_stop", "1")
        key = f"tt_issued_{self.pair.producer}_{self.rank}"
        t0 = time.time()
        while not store_has(key) and not self.finished:
            if time.time() - t0 > self.timeout_s:
                raise EncoderTimeout("producer did not acknowledge the stop request")
            if self._pending is not None or self._announced() > self._posted:
                self._receive()                    # a sample (or the stop header) that was already on its way
            time.sleep(0.005)
        issued = int(st.get(key).decode()) if not self.finished else self.received
        while self.received < issued and not self.finished:
            self._receive()
        if not self.finished:                      # an unfinished stream is closed by a stop header
            self._receive()
        self.finished = True


class WanDistBatchLoader(DistBatchLoader):
    schema = WAN_SCHEMA


class HunyuanDistBatchLoader(DistBatchLoader):
    schema = HUNYUAN_SCHEMA


class OriginBatchLoader:
    """Plain passthrough of a local data iterator (the reference's 'hunyuan origin' loader)."""

    def __init__(self, iterator):
        self.iterator = iterator

    def __iter__(self):
        return self

    def __next__(self):
        return next(self.iterator)


def create_batch_loader(model_name: str, args, iterator=None):
    if iterator is not None and not args.distributed_vae:
        return OriginBatchLoader(iterator)
    kw = dict(timeout_s=float(getattr(args, "encoder_timeout_seconds", 600.0)),
              heartbeat_stale_s=float(getattr(args, "encoder_heartbeat_stale_seconds", 120.0)))
    if "Hunyuan" in model_name:
        return HunyuanDistBatchLoader(args, **kw)
    return WanDistBatchLoader(args, **kw)
