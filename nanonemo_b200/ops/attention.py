"""Causal grouped-query FlashAttention on tcgen05/TMEM (csrc/flash_fwd.cu, csrc/flash_bwd.cu).

``flash_attn(q, k, v)`` takes (B, H, T, hd) / (B, KVH, T, hd) tensors with any strides whose last
dim is contiguous (transposed views of a (B, T, H, hd) projection are the common case) and returns
(B, H, T, hd); ``flash_attn_packed(qkv, H, KVH, hd)`` reads the three operands straight out of the
packed (B, T, (H + 2 KVH) hd) projection and writes (B, T, H hd), and its backward writes dQ, dK, dV
into one packed gradient tensor, so no split / transpose / concat kernels run around attention.
Query head h reads KV head h // (H // KVH) directly (as the reference kernel does,
nanonemo/kernels/cuda/flash_attn.cu:59,72-74). The log-sum-exp per row is saved for backward.
"""

import math

import torch

from nanonemo_b200.ops import _lib
from nanonemo_b200.ops.gemm import status_tensor


def _strides_bthd(t):
    """(sb, st, sh) element strides of a tensor viewed as [B, T, heads, hd]."""
    assert t.stride(-1) == 1, "last dimension must be contiguous"
    return t.stride(0), t.stride(1), t.stride(2)


def fwd_raw(q, k, v, o, scale):
    """q, o: [B, T, H, hd] views; k, v: [B, T, KVH, hd] views (any strides, contiguous last dim)."""
    B, T, H, hd = q.shape
    KVH = k.shape[2]
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    _lib.call("nnb_flash_fwd", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.i32(B), _lib.i32(T),
              _lib.i32(H), _lib.i32(KVH), _lib.i32(hd), *(_lib.i64(s) for s in _strides_bthd(q)),
              *(_lib.i64(s) for s in _strides_bthd(k)), *(_lib.i64(s) for s in _strides_bthd(v)),
              *(_lib.i64(s) for s in _strides_bthd(o)), _lib.f32(scale), _lib.i32(1), _lib.ptr(status_tensor(q.device)),
              _lib.vp(_lib.stream_ptr()))
    return lse


def bwd_raw(q, k, v, o, lse, do, dq, dk, dv, scale, rope_cos=None, rope_sin=None):
    """With `rope_cos` / `rope_sin` (fp32 [T, hd / 2], head_dim 64 only) dQ and dK are returned through the inverse RoPE,
    i.e. as gradients of the projection BEFORE the rotation that produced q and k."""
    B, T, H, hd = q.shape
    KVH = k.shape[2]
    # delta = rowsum(dO * O) is computed inside the launcher's pre-pass kernel
    delta = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    dq_acc = torch.empty((B, T, H, hd), dtype=torch.float32, device=q.device)  # cleared by the kernel's pre-pass
    _lib.call("nnb_flash_bwd", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse),
              _lib.ptr(delta), _lib.ptr(dq_acc), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.i32(B), _lib.i32(T),
              _lib.i32(H), _lib.i32(KVH), _lib.i32(hd), *(_lib.i64(s) for s in _strides_bthd(q)),
              *(_lib.i64(s) for s in _strides_bthd(k)), *(_lib.i64(s) for s in _strides_bthd(v)),
              *(_lib.i64(s) for s in _strides_bthd(o)), *(_lib.i64(s) for s in _strides_bthd(do)),
              *(_lib.i64(s) for s in _strides_bthd(dq)), *(_lib.i64(s) for s in _strides_bthd(dk)),
              *(_lib.i64(s) for s in _strides_bthd(dv)), _lib.f32(scale), _lib.i32(1), _lib.ptr(rope_cos), _lib.ptr(rope_sin),
              _lib.ptr(status_tensor(q.device)), _lib.vp(_lib.stream_ptr()))


def _have_bwd() -> bool:
    return hasattr(_lib.lib(), "nnb_flash_bwd")


def _bwd_via_recompute(q, k, v, do):
    """Gradient by differentiating PyTorch's attention on the same operands ([B, T, heads, hd] views).
    Only used while the library has no backward kernel for the shape."""
    with torch.enable_grad():
        q_, k_, v_ = (t.detach().transpose(1, 2).requires_grad_() for t in (q, k, v))
        group = q_.shape[1] // k_.shape[1]
        out = torch.nn.functional.scaled_dot_product_attention(
            q_, k_.repeat_interleave(group, dim=1), v_.repeat_interleave(group, dim=1), is_causal=True)
        gq, gk, gv = torch.autograd.grad(out, (q_, k_, v_), do.transpose(1, 2))
    return gq.transpose(1, 2), gk.transpose(1, 2), gv.transpose(1, 2)


class _FlashPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, H, KVH, hd):
        B, T, C = qkv.shape
        if qkv.dtype != torch.bfloat16:
            qkv = qkv.to(torch.bfloat16)
        qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
        q = qkv[..., : H * hd].view(B, T, H, hd)
        k = qkv[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd)
        v = qkv[..., (H + KVH) * hd:].view(B, T, KVH, hd)
        o = torch.empty((B, T, H, hd), dtype=qkv.dtype, device=qkv.device)
        scale = 1.0 / math.sqrt(hd)
        lse = fwd_raw(q, k, v, o, scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (H, KVH, hd, scale)
        return o.view(B, T, H * hd)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        H, KVH, hd, scale = ctx.meta
        B, T, C = qkv.shape
        q = qkv[..., : H * hd].view(B, T, H, hd)
        k = qkv[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd)
        v = qkv[..., (H + KVH) * hd:].view(B, T, KVH, hd)
        do = do.reshape(B, T, H, hd)
        do = do if do.stride(-1) == 1 and do.dtype == qkv.dtype else do.to(qkv.dtype).contiguous()
        dqkv = torch.empty_like(qkv)
        dq = dqkv[..., : H * hd].view(B, T, H, hd)
        dk = dqkv[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd)
        dv = dqkv[..., (H + KVH) * hd:].view(B, T, KVH, hd)
        if _have_bwd() and hd in (64, 128):
            bwd_raw(q, k, v, o, lse, do, dq, dk, dv, scale)
        else:
            gq, gk, gv = _bwd_via_recompute(q, k, v, do)
            dq.copy_(gq)
            dk.copy_(gk)
            dv.copy_(gv)
        return dqkv, None, None, None


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        # public layout (B, H, T, hd) -> kernel layout [B, T, H, hd] views (no copies)
        def prep(t):
            t = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
            t = t.transpose(1, 2)
            ok = t.stride(-1) == 1 and all((s * 2) % 16 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0
            return t if ok else t.contiguous()

        ctx.in_dtype = q.dtype
        qt, kt, vt = prep(q), prep(k), prep(v)
        B, T, H, hd = qt.shape
        o = torch.empty((B, T, H, hd), dtype=torch.bfloat16, device=q.device)
        scale = 1.0 / math.sqrt(hd)
        lse = fwd_raw(qt, kt, vt, o, scale)
        ctx.save_for_backward(qt, kt, vt, o, lse)
        ctx.scale = scale
        return o.transpose(1, 2).to(q.dtype)  # (B, H, T, hd) view of a contiguous (B, T, H, hd) buffer

    @staticmethod
    def backward(ctx, do):
        qt, kt, vt, o, lse = ctx.saved_tensors
        B, T, H, hd = qt.shape
        dot = do.transpose(1, 2)
        dot = dot if dot.dtype == torch.bfloat16 and dot.stride(-1) == 1 else dot.to(torch.bfloat16).contiguous()
        if _have_bwd() and hd in (64, 128):
            dq, dk, dv = torch.empty_like(o), torch.empty(kt.shape, dtype=o.dtype, device=o.device), torch.empty(vt.shape, dtype=o.dtype, device=o.device)
            bwd_raw(qt, kt, vt, o, lse, dot, dq, dk, dv, ctx.scale)
        else:
            dq, dk, dv = _bwd_via_recompute(qt, kt, vt, dot)
        return tuple(t.transpose(1, 2).to(ctx.in_dtype) for t in (dq, dk, dv))


def flash_attn_packed(qkv, n_heads, n_kv_heads, head_dim):
    return _FlashPacked.apply(qkv, n_heads, n_kv_heads, head_dim)


def flash_attn(q, k, v):
    return _Flash.apply(q, k, v)
