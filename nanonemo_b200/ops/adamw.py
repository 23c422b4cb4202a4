"""Flat-buffer optimizer kernels (csrc/adamw.cu): squared gradient norm and the fused AdamW step."""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_scratch: dict = {}


def _sumsq_scratch(device):
    key = (device.type, device.index)
    s = _scratch.get(key)
    if s is None:
        s = torch.zeros(_lib.lib().nnb_sumsq_blocks() + 1, dtype=torch.float32, device=device)
        _scratch[key] = s
    return s


def sumsq(x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """sum(x**2) of a contiguous fp32 tensor as a 0-dim fp32 device tensor; summation order is fixed."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = out if out is not None else torch.empty((), dtype=torch.float32, device=x.device)
    _lib.call("nnb_sumsq_f32", _lib.ptr(x), _lib.i64(x.numel()), _lib.ptr(_sumsq_scratch(x.device)), _lib.ptr(out),
              _lib.i32(1 if accumulate else 0), _lib.vp(_lib.stream_ptr()))
    return out


def adamw_flat(p, g, m, v, shadow, decay_flags, *, lr, beta1, beta2, eps, weight_decay, step, grad_norm_sq=None,
               max_norm=None, zero_grad=True):
    n = p.numel()
    _lib.call("nnb_adamw_flat", _lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), _lib.ptr(shadow), _lib.ptr(decay_flags),
              _lib.i64(n), _lib.f32(lr), _lib.f32(beta1), _lib.f32(beta2), _lib.f32(eps), _lib.f32(weight_decay),
              _lib.i32(step), _lib.ptr(grad_norm_sq if max_norm is not None else None),
              _lib.f32(max_norm if max_norm is not None else 0.0), _lib.i32(1 if zero_grad else 0),
              _lib.i32(_CODE[shadow.dtype] if shadow is not None else 1), _lib.vp(_lib.stream_ptr()))
