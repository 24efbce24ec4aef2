"""The allocation-free column-sum entry point (csrc/tt_noalloc.h), called through its exported C
symbol the way a host that cannot allocate device memory would call it.

Such a host (all device memory already handed to another allocator, or a code path where
cudaMalloc's device-wide synchronisation is unacceptable) passes only its own input and output
buffers; the partial sums live in a fixed array inside the library.  The test checks the result
against the ordinary entry point (``tt_colsum``, caller-provided scratch) on calls in a row —
the later ones with smaller problems, so the array still holds the first call's partial sums, one of
them with row chunks that hold no rows at all — and checks that an oversized request and a row
stride smaller than the row are refused with a readable message.  It is collected near the end
so a run that stops at the first failure has already exercised the rest.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from teletron_b200.ops import _lib
from teletron_b200.ops.linear import colsum

MAX_C = 16384


def _symbol():
    L = ctypes.CDLL(str(_lib.lib_file()))
    fn = L.tt_colsum_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    L.tt_last_error.restype = ctypes.c_char_p
    return L, fn


def _call(fn, x, out, accumulate=0):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), x.stride(0), out.data_ptr(), int(out.dtype == torch.float32), accumulate,
              x.shape[0], x.shape[1], stream)


def test_no_alloc_colsum_matches_regular_entry_point_twice():
    L, fn = _symbol()
    torch.manual_seed(0)
    # first call: wide and tall (fills most of the built-in array)
    x1 = torch.randn(5000, 8960, device="cuda").to(torch.bfloat16)
    out1 = torch.empty(8960, dtype=torch.float32, device="cuda")
    assert _call(fn, x1, out1) == 0, L.tt_last_error().decode()
    ref1 = colsum(x1)
    # second call right after: smaller problem on a strided view, bf16 output, accumulate mode
    big = torch.randn(37, 3 * 1536, device="cuda").to(torch.bfloat16)
    x2 = big[:, 1536:3072]
    base = torch.randn(1536, device="cuda").to(torch.bfloat16)
    out2 = base.clone()
    assert _call(fn, x2, out2, accumulate=1) == 0, L.tt_last_error().decode()
    ref2 = (base.float() + colsum(x2)).to(torch.bfloat16)
    # third call: 65 rows split into 64 chunks of 2 rows, so chunks 33..63 hold no rows and must come out as zeros
    # over the first call's partial sums that still sit there
    x3 = torch.randn(65, 8960, device="cuda").to(torch.bfloat16)
    out3 = torch.empty(8960, dtype=torch.float32, device="cuda")
    assert _call(fn, x3, out3) == 0, L.tt_last_error().decode()
    ref3 = colsum(x3)
    torch.cuda.synchronize()
    assert (out3 - ref3).abs().max().item() <= 1e-4 * ref3.abs().max().item()
    assert (out3 - x3.float().sum(0)).abs().max().item() <= 1e-3 * ref3.abs().max().item()
    scale1 = ref1.abs().max().item()
    assert (out1 - ref1).abs().max().item() <= 1e-4 * scale1
    assert (out2.float() - ref2.float()).abs().max().item() <= 2e-2 * ref2.float().abs().max().item()
    # independent fp32 check of the first call
    assert (out1 - x1.float().sum(0)).abs().max().item() <= 1e-3 * scale1


def test_no_alloc_colsum_rejects_oversized_width():
    L, fn = _symbol()
    x = torch.zeros(4, MAX_C + 8, dtype=torch.bfloat16, device="cuda")
    out = torch.full((MAX_C + 8,), 7.0, dtype=torch.float32, device="cuda")
    rc = _call(fn, x, out)
    assert rc != 0
    msg = L.tt_last_error().decode()
    assert "exceeds" in msg and str(MAX_C) in msg
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)  # nothing was launched


def test_no_alloc_colsum_rejects_overlapping_rows():
    L, fn = _symbol()
    x = torch.zeros(8 * 64, dtype=torch.bfloat16, device="cuda")
    out = torch.full((64,), 7.0, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), 32, out.data_ptr(), 1, 0, 8, 64, stream)      # row stride 32 < 64 columns
    assert rc != 0 and "stride" in L.tt_last_error().decode()
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)
