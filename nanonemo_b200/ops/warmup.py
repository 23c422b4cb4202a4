"""Toolchain smoke test: ``c = a + b`` on fp32 tensors through the built library (the counterpart of
the reference's tutorial extension, nanonemo/kernels/cuda/warmup_add.cu)."""

import torch

from nanonemo_b200.ops import _lib


def warmup_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError("warmup_add takes float32 tensors")
    if a.shape != b.shape or not a.is_cuda or not b.is_cuda:
        raise ValueError("warmup_add takes two CUDA tensors of the same shape")
    a, b = a.contiguous(), b.contiguous()
    c = torch.empty_like(a)
    _lib.call("nnb_warmup_add", _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.i64(a.numel()), _lib.vp(_lib.stream_ptr()))
    return c
