"""A cross-rank wait that nobody answers must run out, report where it gave up, and leave the GPU usable."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_with_status_and_context_survives():
    from nanonemo_b200.ops import _lib

    flags = torch.zeros(256, dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    result = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.call("nnb_comm_timeout_probe", _lib.ptr(flags), _lib.ptr(status), _lib.ptr(result), _lib.i32(7), _lib.i32(20000),
              ctypes.c_void_p(_lib.stream_ptr()))
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    st = status.tolist()
    assert result.item() == -1
    assert st[0] == 10 and st[1] == 0 and st[2] == 1 and st[3] == 0 and st[4] == 7  # {phase-0 timeout, rank, silent peer, block, epoch}
    assert flags[0].item() == 7  # the rank's own signal was written
    # the context is intact: ordinary work still runs and a second probe whose flag IS set succeeds
    x = torch.randn(1024, device="cuda")
    assert torch.isfinite((x * 2).sum())
    flags[1] = 9
    status.zero_()
    _lib.call("nnb_comm_timeout_probe", _lib.ptr(flags), _lib.ptr(status), _lib.ptr(result), _lib.i32(9), _lib.i32(20000),
              ctypes.c_void_p(_lib.stream_ptr()))
    torch.cuda.synchronize()
    assert result.item() == 1 and status[0].item() == 0
