"""The allocation-free sum-of-squares entry point, called through its exported C symbol.

For callers that cannot ask for device memory (allocator locked after start-up, code running where
cudaMalloc is not allowed, plain C / ctypes users without a tensor library) the library keeps the
kernel's scratch in a built-in device array. The result must equal the ordinary entry point's,
which takes caller-provided scratch, on two calls in a row (the second call sees the scratch
contents the first one left). Collected last so that a failure here cannot hide other tests.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _noalloc(lib, x, out):
    fn = lib.nnb_sumsq_f32_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    return fn(x.data_ptr(), x.numel(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("n", [4096, 3 * 1024 * 1024 + 17])
def test_noalloc_sumsq_matches_regular_entry_point_twice(n):
    from nanonemo_b200.ops import _lib
    from nanonemo_b200.ops.adamw import sumsq

    lib = _lib.lib()
    torch.manual_seed(n)
    for call in range(2):
        x = torch.randn(n, device="cuda") * (call + 1)
        want = sumsq(x)
        got = torch.full((), -1.0, device="cuda")
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = _noalloc(lib, x, got)
        assert rc == 0, lib.nnb_last_error()
        torch.cuda.synchronize()
        # neither PyTorch's caching allocator nor the driver (cudaMemGetInfo sees every cudaMalloc of the process) gave anything out
        assert torch.cuda.memory_allocated() == before and torch.cuda.mem_get_info()[0] >= free_before
        torch.testing.assert_close(got, want, rtol=1e-5, atol=0)
        torch.testing.assert_close(got, x.double().pow(2).sum().float(), rtol=1e-5, atol=0)


def test_noalloc_rejects_oversized_and_null():
    from nanonemo_b200.ops import _lib

    lib = _lib.lib()
    lib.nnb_last_error.restype = ctypes.c_char_p
    fn = lib.nnb_sumsq_f32_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    x = torch.zeros(256, device="cuda")
    out = torch.zeros((), device="cuda")
    assert fn(x.data_ptr(), (1 << 32) + 1, out.data_ptr(), 0) < 0
    assert b"outside" in lib.nnb_last_error()
    assert fn(None, 16, out.data_ptr(), 0) < 0
    out.fill_(7.0)
    assert fn(None, 0, out.data_ptr(), 0) == 0  # an empty input needs no buffer: the sum is zero
    torch.cuda.synchronize()
    assert out.item() == 0.0
