"""Raw launchers of the SwiGLU activation ``silu(g) * u`` (csrc/elementwise.cu). Backward recomputes the sigmoid from
the saved g and u (reference: nanonemo/kernels/triton/swiglu.py:19-66); gate and up may be the two halves of the fused
gate||up GEMM output (independent row strides). The differentiable operators are registered in ``ops/library.py``
(``swiglu`` on the packed projection, ``swiglu_gu`` on separate tensors)."""

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
