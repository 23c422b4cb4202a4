"""Block-scaled FP8 (MXFP8: e4m3 elements, one e8m0 scale per 32 contraction elements) for the block
linears — this framework's counterpart of the reference's Transformer-Engine shim
(nanonemo/te/__init__.py:20-39: ``te.Linear`` + ``fp8_autocast`` with delayed / current per-tensor
scaling, never run by its authors).

``linear_mxfp8`` quantises the activations, the weights and the output gradients along their contraction
dimensions (csrc/mxfp8.cu: one read of a tensor yields both the row-wise copy and the transposed copy with
their scales) and multiplies the packed bytes on the block-scaled tensor-core path
(``tcgen05.mma.kind::mxf8f6f4.block_scale``, csrc/gemm.cu ``nnb_gemm_mxfp8``: scales staged through shared
memory into tensor memory with ``tcgen05.cp``). Shapes that are not multiples of 128 — and
``NANONEMO_FP8_EMULATE=1`` — take the emulation instead: the same MXFP8-representable values multiplied by
the bf16 GEMM (``fake_quant``), which is also the numerics oracle of the tests. ``fp8_recipe``
(delayed / current) is accepted for config compatibility: block scaling needs no amax history. The LM head
stays bf16, as in the reference.
"""

import os
from contextlib import contextmanager

import torch

from nanonemo_b200.ops import _lib
from nanonemo_b200.ops.gemm import gemm, shadow_of, status_tensor


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


def quantize_mx(x: torch.Tensor, rowwise: bool = True, colwise: bool = False):
    """x [R, C] bf16, R and C multiples of 128 -> (q, sf, qt, sft): q [R, C] e4m3 bytes with blocks along C, qt [C, R] (the
    transpose) with blocks along R, each with its e8m0 scales in the 512-byte-chunk layout the GEMM reads (chunk
    [row / 128][k / 128]; see ``scales_to_plain``). Entries of a pair that was not requested are None."""
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    R, C = x.shape
    dev = x.device
    q = sf = qt = sft = None
    if rowwise:
        q = torch.empty((R, C), dtype=torch.uint8, device=dev)
        sf = torch.empty((R // 128) * (C // 128) * 512, dtype=torch.uint8, device=dev)
    if colwise:
        qt = torch.empty((C, R), dtype=torch.uint8, device=dev)
        sft = torch.empty((C // 128) * (R // 128) * 512, dtype=torch.uint8, device=dev)
    _lib.call("nnb_mxfp8_quantize_sw", _lib.ptr(x), _lib.i64(x.stride(0)), _lib.ptr(q) if rowwise else _lib.vp(None), _lib.i64(C),
              _lib.ptr(sf) if rowwise else _lib.vp(None), _lib.ptr(qt) if colwise else _lib.vp(None), _lib.i64(R),
              _lib.ptr(sft) if colwise else _lib.vp(None), _lib.i32(R), _lib.i32(C), _lib.vp(_lib.stream_ptr()))
    return q, sf, qt, sft


def scales_to_plain(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Chunked scales of a [rows, k] operand -> plain [rows, k / 32] (for tests and debugging)."""
    c = sf.view(rows // 128, k // 128, 32, 4, 4)  # [row chunk, k chunk, row % 32, (row % 128) / 32, k block in chunk]
    return c.permute(0, 3, 2, 1, 4).reshape(rows, k // 32)


def gemm_mxfp8(aq, asf, bq, bsf, out=None, out_dtype=torch.bfloat16, accumulate=False, k_splits=0):
    """(aq [M, K], asf) x (bq [N, K], bsf)^T -> [M, N] bf16 or fp32 on the block-scaled tensor-core path."""
    M, K = aq.shape
    N = bq.shape[0]
    assert bq.shape[1] == K and aq.dtype == bq.dtype == torch.uint8
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype, device=aq.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    _lib.call("nnb_gemm_mxfp8", _lib.ptr(aq), _lib.ptr(asf), _lib.ptr(bq), _lib.ptr(bsf), _lib.ptr(out), _lib.i32(M), _lib.i32(N),
              _lib.i32(K), _lib.i64(aq.stride(0)), _lib.i64(bq.stride(0)), _lib.i64(out.stride(0)),
              _lib.i32(int(out.dtype == torch.float32)), _lib.i32(int(accumulate)), _lib.i32(k_splits), _lib.i32(0),
              _lib.ptr(status_tensor(aq.device)), _lib.vp(_lib.stream_ptr()))
    return out


# Quantised copies of a weight are made once per optimizer step, not once per forward: every micro-batch of the step, and
# the dgrad of every one of them, multiplies by the same bytes. The optimizers of this framework call `weights_changed()`
# after they have rewritten the 16-bit shadow weights; only store-managed weights (they carry `_shadow`) are cached.
_WEIGHT_EPOCH = 0


def weights_changed() -> None:
    global _WEIGHT_EPOCH
    _WEIGHT_EPOCH += 1


def quantized_weight(weight: torch.Tensor, w16: torch.Tensor):
    """(wq, ws, wtq, wts) of `w16` [N, K]: blocks along K for fprop, the transposed copy with blocks along N for dgrad."""
    managed = getattr(weight, "_shadow", None) is w16
    if managed:
        hit = getattr(weight, "_mx_cache", None)
        if hit is not None and hit[0] == _WEIGHT_EPOCH and hit[1] == w16.data_ptr():
            return hit[2]
    q = quantize_mx(w16, True, True)
    if managed:
        weight._mx_cache = (_WEIGHT_EPOCH, w16.data_ptr(), q)
    return q


def _tensor_core_ok(*dims) -> bool:
    return os.environ.get("NANONEMO_FP8_EMULATE", "0") != "1" and all(d % 128 == 0 for d in dims)


class _LinearMXFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        w16 = shadow_of(weight, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        ctx.x_dtype, ctx.real = x.dtype, _tensor_core_ok(x2.shape[0], x2.shape[1], weight.shape[0])
        need_w, need_x = ctx.needs_input_grad[1], ctx.needs_input_grad[0]
        if ctx.real:
            xq, xs, xtq, xts = quantize_mx(x2, True, need_w)           # x along K_in (fprop); x^T along tokens (wgrad)
            wq, ws, wtq, wts = quantized_weight(weight, w16)           # W along K_in (fprop); W^T along N_out (dgrad)
            if not need_x:
                wtq = wts = None
            y = gemm_mxfp8(xq, xs, wq, ws)
            ctx.save_for_backward(weight, *(t for t in (xtq, xts, wtq, wts) if t is not None))
            ctx.flags = (need_w, need_x)
        else:
            y = gemm(fake_quant(x2), fake_quant(w16))  # both quantised along K_in (their contraction dim in fprop)
            ctx.save_for_backward(weight, x2)
            ctx.w16 = w16
        ctx.k_in = x2.shape[-1]
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        weight = ctx.saved_tensors[0]
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        main = getattr(weight, "_main_grad", None)
        direct = main is not None and main.dtype == torch.float32
        if ctx.real:
            rest = list(ctx.saved_tensors[1:])
            need_w, need_x = ctx.flags
            xtq, xts = (rest.pop(0), rest.pop(0)) if need_w else (None, None)
            wtq, wts = (rest.pop(0), rest.pop(0)) if need_x else (None, None)
            dq, ds, dtq, dts = quantize_mx(dy2, need_x, need_w)        # dy along N_out (dgrad); dy^T along tokens (wgrad)
            if need_x:
                dx = gemm_mxfp8(dq, ds, wtq, wts).view(*dy.shape[:-1], ctx.k_in).to(ctx.x_dtype)
            if need_w:
                if direct:
                    gemm_mxfp8(dtq, dts, xtq, xts, out=main, accumulate=True)
                else:
                    dw = gemm_mxfp8(dtq, dts, xtq, xts, out_dtype=torch.float32).to(weight.dtype)
        else:
            x2 = ctx.saved_tensors[1]
            if ctx.needs_input_grad[0]:
                # dgrad contracts over N_out: quantise dy along its rows' N_out, W along N_out (columns of W^T)
                dx = gemm(fake_quant(dy2), fake_quant(ctx.w16.t().contiguous()).t().contiguous(), b_mn=True)
                dx = dx.view(*dy.shape[:-1], x2.shape[-1]).to(ctx.x_dtype)
            if ctx.needs_input_grad[1]:
                # wgrad contracts over tokens: quantise dy^T and x^T along tokens
                dyq = fake_quant(dy2.t().contiguous())  # [N_out, tokens]
                xq = fake_quant(x2.t().contiguous())     # [K_in, tokens]
                if direct:
                    gemm(dyq, xq, out=main, accumulate=True)
                else:
                    dw = gemm(dyq, xq, out_dtype=torch.float32).to(weight.dtype)
        if ctx.needs_input_grad[1] and direct:
            cb = getattr(weight, "_grad_ready_cb", None)
            if cb is not None:
                cb(weight, True)
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
