"""The allocation-free column-sum entry point, called through its exported C symbol.

Callers that may not allocate device memory (plugins inside another runtime's allocator-owned
region, pre-reserved real-time loops, plain C / ctypes hosts without a tensor library) use
`ethb_colsum_noalloc`, which keeps its partial sums in a fixed array inside the library. Its
result must equal the regular launcher's, also on a second call that reuses the same array.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import eth_b200._C as C
    lib = ctypes.CDLL(C.__file__)
    lib.ethb_colsum_noalloc.restype = ctypes.c_int
    lib.ethb_colsum_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.ethb_noalloc_strerror.restype = ctypes.c_char_p
    lib.ethb_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_no_alloc_colsum_matches_regular_entry_point_twice():
    from eth_b200 import ops
    lib = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    # two calls in a row with different shapes: the second reuses the scratch left by the first
    for rows, cols, dt in [(4096, 2048, torch.bfloat16), (777, 512, torch.float16)]:
        x = torch.randn(rows, cols, device="cuda", dtype=dt)
        ref = ops.colsum(x, out_dtype=torch.float32)
        out = torch.empty(cols, device="cuda", dtype=torch.float32)
        before = torch.cuda.memory_allocated()
        rc = lib.ethb_colsum_noalloc(x.data_ptr(), out.data_ptr(), rows, cols, code[dt], 0, 0, stream)
        assert rc == 0, lib.ethb_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel_err(out, ref) < 1e-5
        assert _rel_err(out, x.float().sum(0)) < 1e-5
        assert (out - x.float().sum(0)).abs().max().item() <= 1e-5 * x.float().abs().sum(0).max().item()
        # accumulate on top of an existing value
        acc = torch.full((cols,), 3.0, device="cuda")
        rc = lib.ethb_colsum_noalloc(x.data_ptr(), acc.data_ptr(), rows, cols, code[dt], 0, 1, stream)
        assert rc == 0
        assert _rel_err(acc, ref + 3.0) < 1e-5


def test_no_alloc_colsum_rejects_oversized_and_bad_arguments():
    lib = _lib()
    x = torch.zeros(8, 32768, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(32768, device="cuda")
    rc = lib.ethb_colsum_noalloc(x.data_ptr(), out.data_ptr(), 8, 32768, 2, 0, 0, None)
    assert rc == -2 and b"exceeds" in lib.ethb_noalloc_strerror(rc)
    rc = lib.ethb_colsum_noalloc(x.data_ptr(), out.data_ptr(), 8, 12, 2, 0, 0, None)
    assert rc == -1
    # an input that does not start on a 16-byte boundary is refused before anything is launched
    rc = lib.ethb_colsum_noalloc(x.data_ptr() + 2, out.data_ptr(), 8, 64, 2, 0, 0, None)
    assert rc == -1
