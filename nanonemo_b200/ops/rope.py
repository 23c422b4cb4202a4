"""Fused rotate-half RoPE on Q and K in one launch (csrc/elementwise.cu: rope_packed_kernel).

``rope_qkv`` works on the packed (B, T, (H + 2 KVH) hd) projection: the Q and K heads are rotated,
V is copied through, the result is a new packed tensor that attention reads through strides.
Backward is the same kernel with the sine negated; only the tables are saved (as in the reference,
nanonemo/kernels/triton/rope.py:44-45,87-90). ``apply_rope_qk`` is the (B, T, H, hd) front end.
"""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def rope_packed_raw(x2, out2, cos, sin, T, n_rot_heads, hd, n_copy_cols, sign):
    M = x2.shape[0]
    _lib.call("nnb_rope_packed", _lib.ptr(x2), _lib.ptr(out2), _lib.ptr(cos), _lib.ptr(sin), _lib.i64(M), _lib.i32(T),
              _lib.i32(n_rot_heads), _lib.i32(hd), _lib.i32(n_copy_cols), _lib.i64(x2.stride(0)), _lib.i64(out2.stride(0)),
              _lib.f32(sign), _lib.i32(_CODE[x2.dtype]), _lib.vp(_lib.stream_ptr()))


def _tables(cos, sin, T):
    cos, sin = cos[:T], sin[:T]
    if cos.dtype != torch.float32:
        cos, sin = cos.float(), sin.float()
    return cos.contiguous(), sin.contiguous()


class _RopeQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, H, KVH, hd):
        B, T, C = qkv.shape
        x2 = qkv.reshape(B * T, C)
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        cos, sin = _tables(cos, sin, T)
        out = torch.empty((B * T, C), dtype=qkv.dtype, device=qkv.device)
        rope_packed_raw(x2, out, cos, sin, T, H + KVH, hd, KVH * hd, 1.0)
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
        rope_packed_raw(d2, dx, cos, sin, T, H + KVH, hd, KVH * hd, -1.0)
        return dx.view(B, T, C), None, None, None, None, None


def rope_qkv(qkv, cos, sin, n_heads, n_kv_heads, head_dim):
    return _RopeQKV.apply(qkv, cos, sin, n_heads, n_kv_heads, head_dim)


def apply_rope_qk(q, k, cos, sin):
    """q: (B, T, H, hd), k: (B, T, KVH, hd) with any strides -> contiguous rotated (q, k)."""
    B, T, H, hd = q.shape
    KVH = k.shape[2]
    packed = torch.cat((q.reshape(B, T, H * hd), k.reshape(B, T, KVH * hd)), dim=-1)
    out = _rope_qk_only(packed, cos, sin, H + KVH, hd)
    return out[..., :H * hd].reshape(B, T, H, hd), out[..., H * hd:].reshape(B, T, KVH, hd)


class _RopeHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, n_heads, hd):
        B, T, C = x.shape
        x2 = x.reshape(B * T, C)
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        cos, sin = _tables(cos, sin, T)
        out = torch.empty((B * T, C), dtype=x.dtype, device=x.device)
        rope_packed_raw(x2, out, cos, sin, T, n_heads, hd, 0, 1.0)
        ctx.save_for_backward(cos, sin)
        ctx.meta = (T, n_heads, hd)
        return out.view(B, T, C)

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        T, n_heads, hd = ctx.meta
        B, _, C = dout.shape
        d2 = dout.reshape(B * T, C)
        d2 = d2 if d2.stride(-1) == 1 else d2.contiguous()
        dx = torch.empty((B * T, C), dtype=dout.dtype, device=dout.device)
        rope_packed_raw(d2, dx, cos, sin, T, n_heads, hd, 0, -1.0)
        return dx.view(B, T, C), None, None, None, None


def _rope_qk_only(packed, cos, sin, n_heads, hd):
    return _RopeHeads.apply(packed, cos, sin, n_heads, hd)
