"""Block-scaled FP8 (MXFP8: e4m3 elements, one e8m0 scale per 32 contraction elements) for the block
linears — this framework's counterpart of the reference's Transformer-Engine shim
(nanonemo/te/__init__.py:20-39: ``te.Linear`` + ``fp8_autocast`` with delayed / current per-tensor
scaling, never run by its authors).

What is built: the quantiser kernels (csrc/mxfp8.cu: packed e4m3 + e8m0 output, and a fused
quantise-dequantise) and ``linear_mxfp8``, which multiplies exactly the MXFP8-representable values of
the activations, the weights and the output gradients — each quantised along its contraction
dimension, as a block-scaled tensor-core GEMM would see them — through the bf16 tcgen05 GEMM.
Numerics are therefore those of MXFP8 training; the throughput is that of the bf16 path plus the
quantisers. The ``kind::mxf8f6f4.block_scale`` GEMM that would consume the packed bytes directly is
not built. ``fp8_recipe`` (delayed / current) is accepted for config compatibility: block scaling
needs no amax history. The LM head stays bf16, as in the reference.
"""

from contextlib import contextmanager

import torch

from nanonemo_b200.ops import _lib
from nanonemo_b200.ops.gemm import gemm, shadow_of


def fake_quant(x: torch.Tensor) -> torch.Tensor:
    """x [M, K] bf16 -> the MXFP8 value of every element (blocks of 32 along K), bf16."""
    x2 = x.reshape(-1, x.shape[-1])
    x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=torch.bfloat16, device=x.device)
    _lib.call("nnb_mxfp8_fake_quant", _lib.ptr(x2), _lib.ptr(y), _lib.i64(x2.shape[0]), _lib.i32(x2.shape[1]),
              _lib.i64(x2.stride(0)), _lib.i64(y.stride(0)), _lib.vp(_lib.stream_ptr()))
    return y.view(x.shape)


def quantize(x: torch.Tensor):
    """x [M, K] bf16 -> (e4m3 bytes [M, K] uint8, e8m0 scales [M, K/32] uint8)."""
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    M, K = x2.shape
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((M, K // 32), dtype=torch.uint8, device=x.device)
    _lib.call("nnb_mxfp8_quantize", _lib.ptr(x2), _lib.ptr(q), _lib.ptr(s), _lib.i64(M), _lib.i32(K), _lib.i64(x2.stride(0)),
              _lib.i64(q.stride(0)), _lib.vp(_lib.stream_ptr()))
    return q, s


def dequantize(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    vals = q.view(torch.float8_e4m3fn).float().view(q.shape[0], -1, 32)
    scale = torch.pow(2.0, s.float() - 127.0).unsqueeze(-1)
    return (vals * scale).view(q.shape)


class _LinearMXFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        w16 = shadow_of(weight, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        xq, wq = fake_quant(x2), fake_quant(w16)  # both quantised along K_in (their contraction dim in fprop)
        y = gemm(xq, wq)
        ctx.save_for_backward(x2, weight)
        ctx.w16, ctx.x_dtype = w16, x.dtype
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dgrad contracts over N_out: quantise dy along its rows' N_out, W along N_out (columns of W^T)
            dx = gemm(fake_quant(dy2), fake_quant(ctx.w16.t().contiguous()).t().contiguous(), b_mn=True)
            dx = dx.view(*dy.shape[:-1], x2.shape[-1]).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            # wgrad contracts over tokens: quantise dy^T and x^T along tokens
            dyq = fake_quant(dy2.t().contiguous())  # [N_out, tokens]
            xq = fake_quant(x2.t().contiguous())     # [K_in, tokens]
            main = getattr(weight, "_main_grad", None)
            if main is not None and main.dtype == torch.float32:
                gemm(dyq, xq, out=main, accumulate=True)
                cb = getattr(weight, "_grad_ready_cb", None)
                if cb is not None:
                    cb(weight, True)
            else:
                dw = gemm(dyq, xq, out_dtype=torch.float32).to(weight.dtype)
        return dx, dw


_ENABLED = False


def linear_mxfp8(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """FP8 math only inside ``fp8_context`` (``precision: fp8``); otherwise the plain 16-bit GEMM, which
    is what ``linear_impl: te`` means under ``precision: bf16`` in the reference."""
    if not _ENABLED:
        from nanonemo_b200.ops.gemm import linear_sm100

        return linear_sm100(x, weight)
    return _LinearMXFP8.apply(x, weight)


@contextmanager
def _enabled():
    global _ENABLED
    prev, _ENABLED = _ENABLED, True
    try:
        yield
    finally:
        _ENABLED = prev


def fp8_context(recipe: str = "mxfp8"):
    """Factory of the context manager that wraps the forward pass (cf. the reference's
    ``fp8_context(recipe)``). Block scaling keeps no amax history, so every recipe name maps to the same
    behaviour: the block linears quantise their operands to MXFP8."""
    if recipe not in ("delayed", "current", "mxfp8"):
        raise ValueError(f"unknown fp8 recipe {recipe!r}")
    return _enabled
