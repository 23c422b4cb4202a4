"""Fused residual-add + RMSNorm (csrc/elementwise.cu): ``add_rms_norm(x, delta, w, eps) -> (y, h)``.

``h = x + delta`` is rounded to the dtype of the residual stream before normalising, ``y`` takes the
autocast dtype when autocast is on (else x's dtype), statistics are fp32 — the contract of the
reference operator (nanonemo/kernels/cuda/rmsnorm.py:1-69, rmsnorm.cu:64-167), with bf16 supported.
Backward returns the same tensor for ``dx`` and ``ddelta`` when their dtypes match, and a second
16-bit copy (written by the same kernel) when the residual stream is fp32 and delta is 16-bit.
"""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _y_dtype(x: torch.Tensor, delta) -> torch.dtype:
    if torch.is_autocast_enabled("cuda"):
        return torch.get_autocast_dtype("cuda")
    return delta.dtype if delta is not None else x.dtype


def fwd(x, delta, weight, eps, y_dtype):
    """Raw launcher. x: (..., N) residual dtype; delta same shape or None. Returns (y, h, rstd)."""
    N = x.shape[-1]
    x2 = x.reshape(-1, N)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    M = x2.shape[0]
    d2 = None
    if delta is not None:
        d2 = delta.reshape(-1, N)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
    w = weight if weight.dtype == torch.float32 else weight.float()
    y = torch.empty((M, N), dtype=y_dtype, device=x.device)
    h = torch.empty_like(x2) if d2 is not None else x2
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    dcode = _CODE[d2.dtype] if d2 is not None else _CODE[y_dtype]
    _lib.call("nnb_add_rmsnorm_fwd", _lib.ptr(x2), _lib.ptr(d2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h), _lib.ptr(rstd),
              _lib.i32(M), _lib.i32(N), _lib.f32(eps), _lib.i32(_CODE[x2.dtype]), _lib.i32(dcode),
              _lib.i32(_CODE[y_dtype]), _lib.vp(_lib.stream_ptr()))
    return y.view(*x.shape[:-1], N), h.view(x.shape), rstd


def bwd(dy, h, rstd, weight, dres, delta_dtype, dw_out=None, accumulate=False):
    """Raw launcher. Returns (dx [residual dtype], ddelta [delta dtype or None], dw fp32 [N])."""
    N = h.shape[-1]
    h2 = h.reshape(-1, N)
    M = h2.shape[0]
    dy2 = dy.reshape(-1, N)
    dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
    dr2 = None
    if dres is not None:
        dr2 = dres.reshape(-1, N)
        dr2 = dr2 if dr2.is_contiguous() else dr2.contiguous()
        if dr2.dtype != h2.dtype:
            dr2 = dr2.to(h2.dtype)
    w = weight if weight.dtype == torch.float32 else weight.float()
    dx = torch.empty_like(h2)
    ddelta = None
    if delta_dtype is not None and delta_dtype != h2.dtype:
        ddelta = torch.empty((M, N), dtype=delta_dtype, device=h.device)
    blocks = _lib.lib().nnb_rmsnorm_bwd_blocks()
    partial = torch.empty((blocks, N), dtype=torch.float32, device=h.device)
    dw = dw_out if dw_out is not None else torch.empty(N, dtype=torch.float32, device=h.device)
    dcode = _CODE[delta_dtype] if delta_dtype is not None else _CODE[dy2.dtype]
    _lib.call("nnb_add_rmsnorm_bwd", _lib.ptr(dy2), _lib.ptr(h2), _lib.ptr(rstd), _lib.ptr(w), _lib.ptr(dr2), _lib.ptr(dx),
              _lib.ptr(ddelta), _lib.ptr(dw), _lib.ptr(partial), _lib.i32(M), _lib.i32(N), _lib.i32(_CODE[h2.dtype]),
              _lib.i32(dcode), _lib.i32(_CODE[dy2.dtype]), _lib.i32(1 if accumulate else 0), _lib.vp(_lib.stream_ptr()))
    dx = dx.view(h.shape)
    if delta_dtype is not None and ddelta is None:
        ddelta = dx
    elif ddelta is not None:
        ddelta = ddelta.view(h.shape)
    return dx, ddelta, dw


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        y_dtype = _y_dtype(x, delta)
        if delta is not None and delta.dtype != y_dtype:
            delta = delta.to(y_dtype)
        if x.dtype not in (torch.float32, y_dtype):
            x = x.float()
        y, h, rstd = fwd(x, delta, weight, eps, y_dtype)
        ctx.save_for_backward(h, rstd, weight)
        ctx.delta_dtype = delta.dtype if delta is not None else None
        ctx.mark_non_differentiable(rstd)
        return y, h, rstd

    @staticmethod
    def backward(ctx, dy, dh, _drstd):
        h, rstd, weight = ctx.saved_tensors
        if dy is None:
            dy = torch.zeros(h.shape, dtype=_y_dtype(h, None) if ctx.delta_dtype is None else ctx.delta_dtype, device=h.device)
        main = getattr(weight, "_main_grad", None)
        if main is not None and main.dtype == torch.float32:
            dx, ddelta, _ = bwd(dy, h, rstd, weight, dh, ctx.delta_dtype, dw_out=main, accumulate=True)
            cb = getattr(weight, "_grad_ready_cb", None)
            if cb is not None:
                cb(weight, True)
            dw = None
        else:
            dx, ddelta, dw = bwd(dy, h, rstd, weight, dh, ctx.delta_dtype)
            dw = dw.to(weight.dtype)
        return dx, ddelta, dw, None


def add_rms_norm(x, delta, weight, eps):
    y, h, _ = _AddRMSNorm.apply(x, delta, weight, eps)
    return y, h
