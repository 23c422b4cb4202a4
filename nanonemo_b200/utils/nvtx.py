"""NVTX ranges around the phases of a training step (forward, backward, optimizer, evaluation, checkpoint), so that a
timeline capture (Nsight Systems with ``--capture-range=cudaProfilerApi`` and ``NANONEMO_PROFILE=1``) shows which kernels and
collectives belong to which phase. Off by default: ``NANONEMO_NVTX=1`` turns the ranges on; without CUDA they are no-ops.
The reference has no NVTX annotations (its profiling hooks are the profiler window of nanonemo/train/bench.py:101-119 only).
"""

import os
from contextlib import contextmanager

import torch

_ON = None


def enabled() -> bool:
    global _ON
    if _ON is None:
        _ON = os.environ.get("NANONEMO_NVTX") == "1" and torch.cuda.is_available()
    return _ON


@contextmanager
def span(name: str):
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
