"""Embedding gather / scatter-add for the tied weight (csrc/elementwise.cu).

Forward reads the fp32 master rows and writes the residual-stream dtype. Backward adds each token's
gradient row into the fp32 gradient of the table with 16-byte vector reductions; when the weight
lives in a flat parameter store the rows go straight into the flat gradient buffer (where the fused
linear+cross-entropy already accumulated the head's share) and the parameter is reported ready.
"""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

RESIDUAL_DTYPE = torch.float32  # dtype of the residual stream produced by the sm100 embedding


def fwd_raw(idx, weight, out_dtype):
    flat = idx.reshape(-1)
    flat = flat if flat.dtype == torch.int64 else flat.long()
    flat = flat if flat.is_contiguous() else flat.contiguous()
    V, D = weight.shape
    out = torch.empty((flat.numel(), D), dtype=out_dtype, device=weight.device)
    _lib.call("nnb_embedding_fwd", _lib.ptr(flat), _lib.ptr(weight), _lib.ptr(out), _lib.i64(flat.numel()), _lib.i32(D),
              _lib.i32(V), _lib.i32(_CODE[out_dtype]), _lib.vp(_lib.stream_ptr()))
    return out.view(*idx.shape, D), flat


def bwd_raw(flat_idx, dout, dW):
    V, D = dW.shape
    d2 = dout.reshape(-1, D)
    d2 = d2 if d2.is_contiguous() else d2.contiguous()
    _lib.call("nnb_embedding_bwd", _lib.ptr(flat_idx), _lib.ptr(d2), _lib.ptr(dW), _lib.i64(flat_idx.numel()), _lib.i32(D),
              _lib.i32(V), _lib.i32(_CODE[d2.dtype]), _lib.vp(_lib.stream_ptr()))


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight, out_dtype):
        w = weight if weight.dtype == torch.float32 else weight.float()
        out, flat = fwd_raw(idx, w.contiguous(), out_dtype)
        ctx.save_for_backward(flat, weight)
        return out

    @staticmethod
    def backward(ctx, dout):
        flat, weight = ctx.saved_tensors
        main = getattr(weight, "_main_grad", None)
        if main is not None and main.dtype == torch.float32:
            bwd_raw(flat, dout, main)
            cb = getattr(weight, "_grad_ready_cb", None)
            if cb is not None:
                cb(weight, True)
            return None, None, None
        dW = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        bwd_raw(flat, dout, dW)
        return None, dW.to(weight.dtype), None


def embedding(idx, weight, out_dtype=None):
    return _Embedding.apply(idx, weight, out_dtype or RESIDUAL_DTYPE)
