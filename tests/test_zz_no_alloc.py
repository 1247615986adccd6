"""The allocation-free column-sum entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at all: hosts that gave every
byte of HBM to their own arena, loops that must not hit cudaMalloc's device-wide
synchronisation, plug-ins that only receive buffers.  ``ftk_colsum_bf16_noalloc`` serves
them with a scratch array built into the library.  This test calls it twice in a row (the
second call meets the first call's leftovers in the shared scratch) and checks both results
against the regular entry point, which takes its scratch from the caller.

The file sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from frankentorch_b200.ops import _lib
    lib = _lib.load()
    fn = lib.ftk_colsum_bf16_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    lib.ftk_noalloc_strerror.argtypes = [C.c_int]
    lib.ftk_noalloc_strerror.restype = C.c_char_p
    return lib


def test_noalloc_colsum_matches_regular_entry_point_twice(cuda_device):
    from frankentorch_b200.ops import kernels as K
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    # two different problems back to back: the second reuses scratch the first one filled
    for rows, cols in ((1000, 768), (333, 3072)):
        x = (torch.randn(rows, cols) * 2).to(torch.bfloat16).to(cuda_device)
        want = K.colsum(x)                                    # existing entry point, caller scratch
        got = torch.full((cols,), float("nan"), dtype=torch.float32, device=cuda_device)
        rc = lib.ftk_colsum_bf16_noalloc(x.data_ptr(), got.data_ptr(), rows, cols, x.stride(0), 0, stream)
        assert rc == 0, lib.ftk_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert (got - want).abs().max().item() < 1e-2
        assert (got - x.float().sum(0)).abs().max().item() < 1e-2
        # accumulate mode adds to what is there
        rc = lib.ftk_colsum_bf16_noalloc(x.data_ptr(), got.data_ptr(), rows, cols, x.stride(0), 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert (got - 2 * want).abs().max().item() < 2e-2
    K.check_status()


def test_noalloc_colsum_rejects_oversized_problem(cuda_device):
    lib = _lib()
    x = torch.zeros(8, 8, dtype=torch.bfloat16, device=cuda_device)
    out = torch.zeros(8, dtype=torch.float32, device=cuda_device)
    # ceil(1_000_000/64) * 4096 floats is far beyond the 1 Mi-float scratch: nothing may launch
    rc = lib.ftk_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), 1_000_000, 4096, 4096, 0, None)
    assert rc == -20
    assert b"exceeds the built-in scratch" in lib.ftk_noalloc_strerror(rc)
    assert lib.ftk_colsum_bf16_noalloc(None, out.data_ptr(), 8, 8, 8, 0, None) == -2


def test_noalloc_colsum_rejects_misaligned_pointers_and_too_many_row_blocks(cuda_device):
    """Host-side rejections only: nothing may reach the device for these arguments."""
    lib = _lib()
    x = torch.zeros(16, 16, dtype=torch.bfloat16, device=cuda_device)
    out = torch.zeros(16, dtype=torch.float32, device=cuda_device)
    # a bf16 view that starts at an odd element is 2-byte but not 4-byte aligned
    assert lib.ftk_colsum_bf16_noalloc(x.data_ptr() + 2, out.data_ptr(), 8, 8, 16, 0, None) == -2
    assert lib.ftk_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr() + 2, 8, 8, 16, 0, None) == -2
    # 5,000,000 rows of 2 columns fit the scratch (78,125 * 2 floats) but need 78,125 row blocks
    assert lib.ftk_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), 5_000_000, 2, 2, 1, None) == -20
    # rows near INT_MAX must not overflow the block count
    assert lib.ftk_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), 2**31 - 1, 2, 2, 0, None) == -20
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
