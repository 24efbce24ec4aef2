"""Named NVTX ranges around the framework's fused kernels, off unless a profiling window switches them on
(``--profile``, teletron/train/trainer.py:527-531 in the reference, which relies on ``emit_nvtx`` alone)."""
from __future__ import annotations

import torch

_NVTX_ON = False


def set_nvtx(on: bool) -> bool:
    """Switch the named ranges around the fused kernels on or off (``--profile`` switches them on for the profiled
    steps); returns the previous setting."""
    global _NVTX_ON
    old, _NVTX_ON = _NVTX_ON, bool(on) and torch.cuda.is_available()
    return old


class nvtx_range:
    """``with nvtx_range("qkv_a2a"):`` — an NVTX range when ranges are on, nothing otherwise."""
    __slots__ = ("name", "live")

    def __init__(self, name: str):
        self.name, self.live = name, False

    def __enter__(self):
        if _NVTX_ON:
            torch.cuda.nvtx.range_push(self.name)
            self.live = True
        return self

    def __exit__(self, *exc):
        if self.live:
            torch.cuda.nvtx.range_pop()
        return False
