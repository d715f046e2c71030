"""The allocation-free CRC32 entry point, called the way an outside program would: through the
exported C symbol of libnangila_kernels.so with raw device addresses. It must agree with the ordinary
entry point (which takes its scratch table from the caller) and with zlib, on two calls in a row that
reuse the library's built-in table, and it must refuse buffers larger than that table covers.

Collected last on purpose: a failure here must not hide the result of any other test."""
import ctypes
import os
import zlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "nangila", "libnangila_kernels.so")
    lib = ctypes.CDLL(path)
    lib.nangila_crc32_noalloc.restype = ctypes.c_int
    lib.nangila_crc32_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.nangila_crc32.restype = ctypes.c_int
    lib.nangila_crc32.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.nangila_crc32_scratch_words.restype = ctypes.c_int64
    lib.nangila_crc32_scratch_words.argtypes = [ctypes.c_int64]
    lib.nangila_crc32_noalloc_max_bytes.restype = ctypes.c_int64
    return lib


def test_no_alloc_crc32_agrees_with_the_regular_entry_point_twice():
    lib = _lib()
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out_a = torch.zeros(1, dtype=torch.int32, device="cuda")
    out_b = torch.zeros(1, dtype=torch.int32, device="cuda")
    # a long buffer first, then a short one: the second call finds the first call's leftovers in the table
    for nbytes in (3_000_017, 70_001):
        data = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda")
        words = lib.nangila_crc32_scratch_words(nbytes)
        scratch = torch.empty(words, dtype=torch.int32, device="cuda")
        assert lib.nangila_crc32(data.data_ptr(), nbytes, scratch.data_ptr(), out_a.data_ptr(), stream) == 0
        assert lib.nangila_crc32_noalloc(data.data_ptr(), nbytes, out_b.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        a = int(out_a.item()) & 0xFFFFFFFF
        b = int(out_b.item()) & 0xFFFFFFFF
        assert a == b == zlib.crc32(data.cpu().numpy().tobytes())


def test_no_alloc_crc32_limits():
    lib = _lib()
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.full((1,), 123, dtype=torch.int32, device="cuda")
    limit = lib.nangila_crc32_noalloc_max_bytes()
    assert limit == 64 << 20
    tiny = torch.zeros(16, dtype=torch.uint8, device="cuda")
    # one byte over the limit is refused before anything is queued (cudaErrorInvalidValue == 1)
    assert lib.nangila_crc32_noalloc(tiny.data_ptr(), limit + 1, out.data_ptr(), stream) == 1
    torch.cuda.synchronize()
    assert int(out.item()) == 123
    # an empty buffer hashes to 0
    assert lib.nangila_crc32_noalloc(None, 0, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(out.item()) == 0
