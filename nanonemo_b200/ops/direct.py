"""Direct ``autograd.Function`` variants of the weightless operators (SwiGLU, RoPE, FlashAttention on the packed projection)
for the trainer's engine.

They launch exactly the kernels the registered operators in ``ops/library.py`` launch; what they skip is the dispatcher round
trip of a Python ``torch.library.custom_op`` (tens of microseconds per call, forward and backward). An eager training step of
the 114M model is 300 launches in 20-35 ms, and under tensor parallelism the host is the bottleneck, so the engine — any run
that owns a flat parameter store, see ``enable()`` — takes these; everything else (plain modules, ``torch.compile``,
``opcheck``) takes the registered operators. Contracts: nanonemo/kernels/triton/{swiglu,rope}.py,
nanonemo/kernels/cuda/flash_attn.py.
"""

import math

import torch

from nanonemo_b200.ops import attention, rope, swiglu_act

ENABLED = False


def enable(on: bool = True) -> None:
    """Called by the flat parameter stores: from then on ``nanonemo_b200.ops`` routes the weightless sm100 operators here."""
    global ENABLED
    ENABLED = on


class _SwiGLUPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F = gu.shape[-1] // 2
        gu2 = swiglu_act._rows(gu)
        out = torch.empty((gu2.shape[0], F), dtype=gu.dtype, device=gu.device)
        swiglu_act.fwd_raw(gu2[:, :F], gu2[:, F:], out)
        ctx.save_for_backward(gu2)
        return out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dy):
        (gu2,) = ctx.saved_tensors
        F = gu2.shape[-1] // 2
        dgu = torch.empty_like(gu2)
        swiglu_act.bwd_raw(swiglu_act._rows(dy), gu2[:, :F], gu2[:, F:], dgu[:, :F], dgu[:, F:])
        return dgu.view(*dy.shape[:-1], 2 * F)


class _RopeQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, H, KVH, hd):
        B, T, C = qkv.shape
        x2 = qkv.reshape(B * T, C)
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        out = torch.empty((B * T, C), dtype=qkv.dtype, device=qkv.device)
        rope.rope_packed_raw(x2, out, cos, sin, T, H + KVH, hd, KVH * hd, 1.0)
        ctx.save_for_backward(cos, sin)
        ctx.meta = (T, H, KVH, hd)
        return out.view(B, T, C)

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        T, H, KVH, hd = ctx.meta
        B, _, C = dout.shape
        d2 = dout.reshape(B * T, C)
        d2 = d2 if d2.stride(-1) == 1 else d2.contiguous()
        dx = torch.empty((B * T, C), dtype=dout.dtype, device=dout.device)
        rope.rope_packed_raw(d2, dx, cos, sin, T, H + KVH, hd, KVH * hd, -1.0)
        return dx.view(B, T, C), None, None, None, None, None


def _split(t, B, T, H, KVH, hd):
    return t[..., : H * hd].view(B, T, H, hd), t[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd), t[..., (H + KVH) * hd:].view(B, T, KVH, hd)


class _FlashPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, H, KVH, hd):
        B, T, _ = qkv.shape
        qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
        q, k, v = _split(qkv, B, T, H, KVH, hd)
        o = torch.empty((B, T, H, hd), dtype=qkv.dtype, device=qkv.device)
        scale = 1.0 / math.sqrt(hd)
        lse = attention.fwd_raw(q, k, v, o, scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (H, KVH, hd, scale)
        return o.view(B, T, H * hd)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        H, KVH, hd, scale = ctx.meta
        B, T, _ = qkv.shape
        do = do.reshape(B, T, H, hd)
        do = do if do.stride(-1) == 1 and do.dtype == qkv.dtype else do.to(qkv.dtype).contiguous()
        dqkv = torch.empty_like(qkv)
        attention.bwd_raw(*_split(qkv, B, T, H, KVH, hd), o, lse, do, *_split(dqkv, B, T, H, KVH, hd), scale)
        return dqkv, None, None, None


def swiglu_packed(gu):
    return _SwiGLUPacked.apply(gu)


def rope_qkv(qkv, cos, sin, n_heads, n_kv_heads, head_dim):
    return _RopeQKV.apply(qkv, cos, sin, n_heads, n_kv_heads, head_dim)


def flash_attn_packed(qkv, n_heads, n_kv_heads, head_dim):
    return _FlashPacked.apply(qkv, n_heads, n_kv_heads, head_dim)
