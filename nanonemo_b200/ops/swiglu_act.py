"""SwiGLU activation ``silu(g) * u`` (csrc/elementwise.cu). Backward recomputes the sigmoid from the
saved g and u (reference: nanonemo/kernels/triton/swiglu.py:19-66). ``swiglu_packed`` reads gate and
up from the two halves of the fused gate||up GEMM output without splitting it."""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _rows(t):
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(-1) == 1 else t2.contiguous()


def fwd_raw(g2, u2, out2):
    M, F = out2.shape
    _lib.call("nnb_swiglu_fwd", _lib.ptr(g2), _lib.ptr(u2), _lib.ptr(out2), _lib.i64(M), _lib.i32(F), _lib.i64(g2.stride(0)),
              _lib.i64(u2.stride(0)), _lib.i64(out2.stride(0)), _lib.i32(_CODE[out2.dtype]), _lib.vp(_lib.stream_ptr()))


def bwd_raw(dy2, g2, u2, dg2, du2):
    M, F = dy2.shape
    _lib.call("nnb_swiglu_bwd", _lib.ptr(dy2), _lib.ptr(g2), _lib.ptr(u2), _lib.ptr(dg2), _lib.ptr(du2), _lib.i64(M),
              _lib.i32(F), _lib.i64(dy2.stride(0)), _lib.i64(g2.stride(0)), _lib.i64(u2.stride(0)), _lib.i64(dg2.stride(0)),
              _lib.i64(du2.stride(0)), _lib.i32(_CODE[dy2.dtype]), _lib.vp(_lib.stream_ptr()))


class _SwiGLUPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F = gu.shape[-1] // 2
        gu2 = _rows(gu)
        out = torch.empty((gu2.shape[0], F), dtype=gu.dtype, device=gu.device)
        fwd_raw(gu2[:, :F], gu2[:, F:], out)
        ctx.save_for_backward(gu2)
        return out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dy):
        (gu2,) = ctx.saved_tensors
        F = gu2.shape[-1] // 2
        dy2 = _rows(dy)
        dgu = torch.empty_like(gu2)
        bwd_raw(dy2, gu2[:, :F], gu2[:, F:], dgu[:, :F], dgu[:, F:])
        return dgu.view(*dy.shape[:-1], 2 * F)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g2, u2 = _rows(g), _rows(u)
        out = torch.empty((g2.shape[0], g2.shape[1]), dtype=g.dtype, device=g.device)
        fwd_raw(g2, u2, out)
        ctx.save_for_backward(g2, u2)
        return out.view(g.shape)

    @staticmethod
    def backward(ctx, dy):
        g2, u2 = ctx.saved_tensors
        dy2 = _rows(dy)
        dg = torch.empty((g2.shape[0], g2.shape[1]), dtype=g2.dtype, device=g2.device)
        du = torch.empty_like(dg)
        bwd_raw(dy2, g2, u2, dg, du)
        return dg.view(dy.shape), du.view(dy.shape)


def swiglu_packed(gu):
    return _SwiGLUPacked.apply(gu)


def swiglu(g, u):
    if u.dtype != g.dtype:
        u = u.to(g.dtype)
    return _SwiGLU.apply(g, u)
