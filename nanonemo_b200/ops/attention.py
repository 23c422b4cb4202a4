"""Causal grouped-query FlashAttention on tcgen05/TMEM (csrc/flash_fwd.cu, csrc/flash_bwd.cu).

Raw launchers; the differentiable operators are registered in ``ops/library.py``: ``flash_attn(q, k, v)`` takes
(B, H, T, hd) / (B, KVH, T, hd) tensors with any strides whose last dim is contiguous (transposed views of a
(B, T, H, hd) projection are the common case) and returns (B, H, T, hd); ``flash_attn_packed(qkv, H, KVH, hd)`` reads
the three operands straight out of the packed (B, T, (H + 2 KVH) hd) projection and writes (B, T, H hd), and its
backward writes dQ, dK, dV into one packed gradient tensor, so no split / transpose / concat kernels run around attention.
Operands are bf16 or fp16 (one dtype for all of them; scores, softmax and every accumulator are fp32 either way).
Query head h reads KV head h // (H // KVH) directly (as the reference kernel does,
nanonemo/kernels/cuda/flash_attn.cu:59,72-74). The log-sum-exp per row is saved for backward.
"""

import math

import torch

from nanonemo_b200.ops import _lib
from nanonemo_b200.ops.gemm import status_tensor


_CODE = {torch.bfloat16: 1, torch.float16: 2}


def _dtype_code(*tensors):
    """bf16 or fp16, the same for every operand (the tensor-core instruction takes one 16-bit format for A and B)."""
    dt = tensors[0].dtype
    if dt not in _CODE or any(t.dtype != dt for t in tensors):
        raise TypeError(f"attention kernels take bf16 or fp16 operands of one dtype, got {[str(t.dtype) for t in tensors]}")
    return _CODE[dt]


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
              *(_lib.i64(s) for s in _strides_bthd(o)), _lib.f32(scale), _lib.i32(_dtype_code(q, k, v, o)),
              _lib.ptr(status_tensor(q.device)), _lib.vp(_lib.stream_ptr()))
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
              *(_lib.i64(s) for s in _strides_bthd(dv)), _lib.f32(scale), _lib.i32(_dtype_code(q, k, v, o, do, dq, dk, dv)),
              _lib.ptr(rope_cos), _lib.ptr(rope_sin),
              _lib.ptr(status_tensor(q.device)), _lib.vp(_lib.stream_ptr()))
