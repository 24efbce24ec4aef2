"""Multi-process test harness: run ``fn(rank, world, *args)`` in `world` spawned processes with a
gloo (CPU) or nccl process group on 127.0.0.1, collect each rank's return value."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _pack(o):
    """Tensors travel by value (numpy), not by shared-memory handle, so a worker may exit at once."""
    if torch.is_tensor(o):
        return ("__tensor__", o.detach().cpu().numpy())
    if isinstance(o, (list, tuple)):
        return type(o)(_pack(x) for x in o)
    if isinstance(o, dict):
        return {k: _pack(v) for k, v in o.items()}
    return o


def _unpack(o):
    if isinstance(o, tuple) and len(o) == 2 and isinstance(o[0], str) and o[0] == "__tensor__":
        return torch.from_numpy(o[1])
    if isinstance(o, (list, tuple)):
        return type(o)(_unpack(x) for x in o)
    if isinstance(o, dict):
        return {k: _unpack(v) for k, v in o.items()}
    return o


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, queue):
    import faulthandler

    if os.environ.get("TT_TEST_HANG_DUMP"):
        faulthandler.dump_traceback_later(float(os.environ["TT_TEST_HANG_DUMP"]), exit=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank % torch.cuda.device_count())
        dist.init_process_group(backend, rank=rank, world_size=world)
        out = fn(rank, world, *args)
        queue.put((rank, "ok", _pack(out)))
    except Exception:
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn, world: int, *args, backend: str = "gloo", timeout: float = 300.0):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = queue.get(timeout=timeout)
            if status != "ok":
                raise RuntimeError(f"rank {rank} failed:\n{payload}")
            results[rank] = _unpack(payload)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    return [results[r] for r in range(world)]
