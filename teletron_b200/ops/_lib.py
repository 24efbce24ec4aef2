"""ctypes binding of the native sm_100a library.

The library is built in-tree by ``teletron_b200.build_ext`` and exposes C symbols that
take raw device pointers and a stream handle.  On a machine with a GPU a missing
library is an error (the kernels are the product, there is no silent fallback); on a
CPU-only machine ``available()`` is False and the pure-PyTorch reference ops are used.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LOCK = threading.Lock()
_LIB = None
_STATUS: dict[int, torch.Tensor] = {}

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_uint = ctypes.c_uint


def lib_file() -> Path:
    return Path(__file__).resolve().parent.parent / "_C" / "libtt_b200.so"


def has_gpu() -> bool:
    return torch.cuda.is_available()


def available() -> bool:
    """True when kernels can run: a CUDA device and the built library."""
    return has_gpu() and (lib_file().exists() or os.environ.get("TT_B200_AUTOBUILD") == "1")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            path = lib_file()
            if not path.exists():
                if os.environ.get("TT_B200_AUTOBUILD") == "1":
                    from ..build_ext import build

                    build()
                else:
                    raise RuntimeError(
                        f"native library {path} is missing; run `python -m teletron_b200.build_ext` "
                        "(or __graft_entry__.build()) before using the CUDA ops"
                    )
            L = ctypes.CDLL(str(path))
            L.tt_last_error.restype = ctypes.c_char_p
            L.tt_launch_count.restype = ctypes.c_longlong
            _LIB = L
    return _LIB


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().tt_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed (rc={rc}): {msg}")


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32[4] word that kernels write when a bounded wait runs out."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _STATUS[idx] = t
    return t


# status codes written by the kernels (csrc/tt_common.cuh): high byte = who gave up, low byte = which wait / peer
_STATUS_ROLES = {0x100: "a TMA producer warp waiting for a free stage", 0x200: "the MMA-issuing warp",
                 0x300: "an epilogue warp waiting for an accumulator",
                 0x400: "a softmax / elementwise warp waiting for a tensor-memory tile",
                 0x500: "a peer barrier waiting for rank", 0x600: "a kernel whose dynamic shared memory is misaligned"}


def describe_status(code: int) -> str:
    """Readable form of a status word value, e.g. 0x503 -> the peer barrier gave up waiting for rank 3."""
    if code == 0:
        return "ok"
    role, detail = code & ~0xFF, code & 0xFF
    what = _STATUS_ROLES.get(role)
    if what is None:
        return f"unknown status 0x{code:x}"
    if role == 0x500:
        return f"{what} {detail} ran out of its time budget"
    if role == 0x600:
        return what
    return f"{what} ran out of its time budget (wait #{detail})"


def check_status(device: torch.device | None = None) -> None:
    """Raise if any kernel recorded a timed-out wait since the last check (one D2H read)."""
    t = status_word(device)
    code = int(t[0].item())
    if code != 0:
        t.zero_()
        raise RuntimeError(f"a device-side wait gave up (status 0x{code:x}: {describe_status(code)}); "
                           "results of this step are invalid")


def launch_count() -> int:
    """Kernels launched by the native library in this process so far."""
    return int(lib().tt_launch_count()) if lib_file().exists() else 0
