"""Block-level operators whose elementwise work rides in a GEMM epilogue (csrc/gemm2.cu) or in the attention
backward (csrc/flash_bwd.cu) instead of being a pass over HBM of its own:

``qkv_rope_attention(x, wqkv, cos, sin, H, KVH, hd)``
    packed QKV projection with RoPE applied to the query / key heads in the GEMM epilogue, causal GQA FlashAttention
    on the packed result, and in backward the inverse rotation applied to dQ (in the fp32 -> bf16 conversion of the dQ
    accumulator) and dK (in the kernel's final epilogue), followed by the projection's dgrad / wgrad GEMMs.
``linear_swiglu(x, w_gu)``
    gate||up projection whose epilogue also writes ``silu(gate) * up``; the projection is kept for backward, which
    recomputes the sigmoid from it (as nanonemo/kernels/triton/swiglu.py:45-66 does).
``mlp_swiglu(x, w_gu, w_down)``
    the whole feed-forward as one autograd node, so that the backward of the activation can ride in the epilogue of the
    down projection's input-gradient GEMM: d(gate) | d(up) leave tensor memory directly and the gradient of the
    activation is never written to HBM (the reference runs linear backward, then the SwiGLU backward kernel,
    nanonemo/kernels/triton/swiglu.py:45-90).

Each falls back, operator by operator, to the plain GEMM followed by the stand-alone kernel when the CTA-pair GEMM does
not serve the shape (fewer than 256 rows, d_ff not a multiple of 128, head_dim other than 64 / 128), so results do not
depend on which route ran. The reference composes the same math from separate kernels (nanonemo/model/layers.py:97-138).
"""

import math
import os

import torch

from nanonemo_b200.ops import attention, rope, swiglu_act
from nanonemo_b200.ops.gemm import (_rowmajor2d, compute_dtype, gemm, gemm_rope, gemm_swiglu, gemm_swiglu_bwd, linear_backward,
                                    shadow_of)


def _rows16(x, dt):
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype != dt:
        x2 = x2.to(dt)
    return _rowmajor2d(x2)


def _split(qkv, B, T, H, KVH, hd):
    return (qkv[..., : H * hd].view(B, T, H, hd), qkv[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd),
            qkv[..., (H + KVH) * hd:].view(B, T, KVH, hd))


class _QKVRopeAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cos, sin, H, KVH, hd):
        B, T, _ = x.shape
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        x2 = _rows16(x, dt)
        cos_t, sin_t = rope._tables(cos, sin, T)
        rot_cols = (H + KVH) * hd
        gather = getattr(weight, "_gather_in_gemm", None)
        if gather is not None:
            # FSDP: this GEMM kernel also all-gathers the block's parameters (the weight itself first), see parallel/fsdp.py
            qkv = gather(x2, weight)
        else:
            qkv = gemm_rope(x2, w16, cos_t, sin_t, T, rot_cols, hd)
        if qkv is None or gather is not None:
            if qkv is None:
                qkv = gemm(x2, w16)
            rope.rope_packed_raw(qkv, qkv, cos_t, sin_t, T, H + KVH, hd, 0, 1.0)  # rotates Q and K in place, V untouched
        qkv = qkv.view(B, T, -1)
        q, k, v = _split(qkv, B, T, H, KVH, hd)
        o = torch.empty((B, T, H, hd), dtype=dt, device=x.device)
        scale = 1.0 / math.sqrt(hd)
        lse = attention.fwd_raw(q, k, v, o, scale)
        ctx.save_for_backward(x2, weight, qkv, o, lse, cos_t, sin_t)
        ctx.w16, ctx.meta, ctx.x_shape, ctx.x_dtype = w16, (H, KVH, hd, scale), x.shape, x.dtype
        return o.view(B, T, H * hd)

    @staticmethod
    def backward(ctx, do):
        x2, weight, qkv, o, lse, cos_t, sin_t = ctx.saved_tensors
        H, KVH, hd, scale = ctx.meta
        B, T, _ = qkv.shape
        q, k, v = _split(qkv, B, T, H, KVH, hd)
        do = do.reshape(B, T, H, hd)
        do = do if do.stride(-1) == 1 and do.dtype == qkv.dtype else do.to(qkv.dtype).contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _split(dqkv, B, T, H, KVH, hd)
        # the 128 x 128 backward kernel (head_dim 64) un-rotates dQ and dK itself; otherwise one in-place pass does
        in_kernel = hd == 64 and not os.environ.get("NANONEMO_FLASH_BWD", "").startswith("t")
        if in_kernel:
            attention.bwd_raw(q, k, v, o, lse, do, dq, dk, dv, scale, rope_cos=cos_t, rope_sin=sin_t)
        else:
            attention.bwd_raw(q, k, v, o, lse, do, dq, dk, dv, scale)
            d2 = dqkv.view(B * T, -1)
            rope.rope_packed_raw(d2, d2, cos_t, sin_t, T, H + KVH, hd, 0, -1.0)
        dx, dw = linear_backward(dqkv.view(B * T, -1), x2, weight, ctx.w16, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if dx is not None:
            dx = dx.view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, dw, None, None, None, None, None


def qkv_rope_attention(x, weight, cos, sin, n_heads, n_kv_heads, head_dim):
    """x: (B, T, d); weight: [(H + 2 KVH) hd, d] (fp32 master or 16-bit) -> attention output (B, T, H hd), bf16 compute."""
    return _QKVRopeAttention.apply(x, weight, cos, sin, n_heads, n_kv_heads, head_dim)


class _LinearSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        x2 = _rows16(x, dt)
        F = weight.shape[0] // 2
        fused = gemm_swiglu(x2, w16)
        if fused is None:
            gu = gemm(x2, w16)
            act = torch.empty((x2.shape[0], F), dtype=dt, device=x.device)
            swiglu_act.fwd_raw(gu[:, :F], gu[:, F:], act)
        else:
            gu, act = fused
        ctx.save_for_backward(x2, weight, gu)
        ctx.w16, ctx.x_shape, ctx.x_dtype = w16, x.shape, x.dtype
        return act.view(*x.shape[:-1], F)

    @staticmethod
    def backward(ctx, dact):
        x2, weight, gu = ctx.saved_tensors
        F = gu.shape[1] // 2
        d2 = swiglu_act._rows(dact)
        if d2.dtype != gu.dtype:
            d2 = d2.to(gu.dtype)
        dgu = torch.empty_like(gu)
        swiglu_act.bwd_raw(d2, gu[:, :F], gu[:, F:], dgu[:, :F], dgu[:, F:])
        dx, dw = linear_backward(dgu, x2, weight, ctx.w16, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if dx is not None:
            dx = dx.view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, dw


def linear_swiglu(x, weight):
    """x: (..., d); weight: [2 F, d], gate rows first -> silu(x Wg^T) * (x Wu^T), shape (..., F)."""
    return _LinearSwiGLU.apply(x, weight)


FUSE_SWIGLU_BWD = os.environ.get("NANONEMO_FUSE_SWIGLU_BWD", "1") != "0"


class _MLPSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_gu, w_down):
        dt = compute_dtype()
        w16_gu, w16_down = shadow_of(w_gu, dt), shadow_of(w_down, dt)
        x2 = _rows16(x, dt)
        F = w_gu.shape[0] // 2
        fused = gemm_swiglu(x2, w16_gu)
        if fused is None:
            gu = gemm(x2, w16_gu)
            act = torch.empty((x2.shape[0], F), dtype=dt, device=x.device)
            swiglu_act.fwd_raw(gu[:, :F], gu[:, F:], act)
        else:
            gu, act = fused
        y = gemm(act, w16_down)
        ctx.save_for_backward(x2, w_gu, w_down, gu, act)
        ctx.w16, ctx.x_shape, ctx.x_dtype = (w16_gu, w16_down), x.shape, x.dtype
        return y.view(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w_gu, w_down, gu, act = ctx.saved_tensors
        w16_gu, w16_down = ctx.w16
        F = gu.shape[1] // 2
        dy2 = _rows16(dy, gu.dtype)
        dgu = gemm_swiglu_bwd(dy2, w16_down, gu) if FUSE_SWIGLU_BWD else None
        if dgu is None:
            dact = gemm(dy2, w16_down, b_mn=True)
            dgu = torch.empty_like(gu)
            swiglu_act.bwd_raw(dact, gu[:, :F], gu[:, F:], dgu[:, :F], dgu[:, F:])
        _, dw_down = linear_backward(dy2, act, w_down, w16_down, False, ctx.needs_input_grad[2])
        dx, dw_gu = linear_backward(dgu, x2, w_gu, w16_gu, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if dx is not None:
            dx = dx.view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, dw_gu, dw_down


def mlp_swiglu(x, w_gu, w_down):
    """x: (..., d); w_gu: [2 F, d] (gate rows first); w_down: [d, F] -> down(silu(x Wg^T) * (x Wu^T)), shape (..., d)."""
    return _MLPSwiGLU.apply(x, w_gu, w_down)
