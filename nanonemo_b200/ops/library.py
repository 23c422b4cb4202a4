"""``torch.library`` registration of the sm100 operators: schema + fake (meta) implementation +
autograd formula for each, so they compose with ``torch.compile(fullgraph=True)``, ``opcheck`` and
functional transforms — the binding layer of the reference (nanonemo/kernels/cuda/rmsnorm.py:1-69,
flash_attn.py:1-60: ``custom_op`` + ``register_fake`` + ``register_autograd``), on top of the
ahead-of-time built library instead of a per-process JIT.

The model's hot path calls the ``autograd.Function`` classes in the sibling modules directly (no
dispatcher round trip); the operators here call the same raw launchers and are the public,
composable surface:

    torch.ops.nanonemo_b200.add_rms_norm(x, delta, weight, eps)        -> (y, h)
    torch.ops.nanonemo_b200.swiglu(gu)                                 -> act
    torch.ops.nanonemo_b200.rope_qkv(qkv, cos, sin, H, KVH, hd)        -> qkv_rot
    torch.ops.nanonemo_b200.flash_attn_packed(qkv, H, KVH, hd)         -> (o, lse)
    torch.ops.nanonemo_b200.linear(x, w16)                             -> y
"""

import math

import torch
from torch import Tensor

from nanonemo_b200.ops import attention, gemm as gemm_mod, rmsnorm, rope, swiglu_act

NS = "nanonemo_b200"


# ----------------------------------------------------------------------------- add + RMSNorm
@torch.library.custom_op(f"{NS}::add_rms_norm", mutates_args=(), device_types="cuda")
def add_rms_norm(x: Tensor, delta: Tensor, weight: Tensor, eps: float) -> tuple[Tensor, Tensor, Tensor]:
    y, h, rstd = rmsnorm.fwd(x, delta, weight, eps, delta.dtype)
    return y, h, rstd


@add_rms_norm.register_fake
def _(x, delta, weight, eps):
    return torch.empty_like(delta, memory_format=torch.contiguous_format), torch.empty_like(x, memory_format=torch.contiguous_format), \
        x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32)


@torch.library.custom_op(f"{NS}::add_rms_norm_bwd", mutates_args=(), device_types="cuda")
def add_rms_norm_bwd(dy: Tensor, dh: Tensor, h: Tensor, rstd: Tensor, weight: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    dx, ddelta, dw = rmsnorm.bwd(dy, h, rstd, weight, dh, dy.dtype)
    return dx, ddelta if ddelta is not dx else dx.clone(), dw


@add_rms_norm_bwd.register_fake
def _(dy, dh, h, rstd, weight):
    return torch.empty_like(h), torch.empty_like(dy), weight.new_empty(weight.shape, dtype=torch.float32)


def _arn_setup(ctx, inputs, output):
    _, _, weight, _ = inputs
    _, h, rstd = output
    ctx.save_for_backward(h, rstd, weight)


def _arn_backward(ctx, dy, dh, _drstd):
    h, rstd, weight = ctx.saved_tensors
    dy = dy.contiguous() if dy is not None else torch.zeros(h.shape, dtype=torch.bfloat16, device=h.device)
    dh = dh.contiguous() if dh is not None else torch.zeros_like(h)
    dx, ddelta, dw = add_rms_norm_bwd(dy, dh, h, rstd, weight)
    return dx, ddelta, dw.to(weight.dtype), None


add_rms_norm.register_autograd(_arn_backward, setup_context=_arn_setup)


# ----------------------------------------------------------------------------- SwiGLU (packed gate || up)
@torch.library.custom_op(f"{NS}::swiglu", mutates_args=(), device_types="cuda")
def swiglu(gu: Tensor) -> Tensor:
    F = gu.shape[-1] // 2
    gu2 = swiglu_act._rows(gu)
    out = torch.empty((gu2.shape[0], F), dtype=gu.dtype, device=gu.device)
    swiglu_act.fwd_raw(gu2[:, :F], gu2[:, F:], out)
    return out.view(*gu.shape[:-1], F)


@swiglu.register_fake
def _(gu):
    return gu.new_empty((*gu.shape[:-1], gu.shape[-1] // 2))


@torch.library.custom_op(f"{NS}::swiglu_bwd", mutates_args=(), device_types="cuda")
def swiglu_bwd(dy: Tensor, gu: Tensor) -> Tensor:
    F = gu.shape[-1] // 2
    gu2, dy2 = swiglu_act._rows(gu), swiglu_act._rows(dy)
    dgu = torch.empty((gu2.shape[0], 2 * F), dtype=gu.dtype, device=gu.device)
    swiglu_act.bwd_raw(dy2, gu2[:, :F], gu2[:, F:], dgu[:, :F], dgu[:, F:])
    return dgu.view(gu.shape)


@swiglu_bwd.register_fake
def _(dy, gu):
    return torch.empty_like(gu, memory_format=torch.contiguous_format)


swiglu.register_autograd(lambda ctx, dy: swiglu_bwd(dy.contiguous(), ctx.saved_tensors[0]),
                         setup_context=lambda ctx, inputs, output: ctx.save_for_backward(inputs[0]))


# ----------------------------------------------------------------------------- RoPE on the packed projection
@torch.library.custom_op(f"{NS}::rope_qkv", mutates_args=(), device_types="cuda")
def rope_qkv(qkv: Tensor, cos: Tensor, sin: Tensor, n_heads: int, n_kv_heads: int, head_dim: int, sign: float = 1.0) -> Tensor:
    B, T, C = qkv.shape
    x2 = qkv.reshape(B * T, C)
    x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
    c, s = rope._tables(cos, sin, T)
    out = torch.empty((B * T, C), dtype=qkv.dtype, device=qkv.device)
    rope.rope_packed_raw(x2, out, c, s, T, n_heads + n_kv_heads, head_dim, n_kv_heads * head_dim, sign)
    return out.view(B, T, C)


@rope_qkv.register_fake
def _(qkv, cos, sin, n_heads, n_kv_heads, head_dim, sign=1.0):
    return torch.empty_like(qkv, memory_format=torch.contiguous_format)


def _rope_setup(ctx, inputs, output):
    _, cos, sin, H, KVH, hd, sign = inputs
    ctx.save_for_backward(cos, sin)
    ctx.meta = (H, KVH, hd, sign)


def _rope_backward(ctx, dout):
    cos, sin = ctx.saved_tensors
    H, KVH, hd, sign = ctx.meta
    return rope_qkv(dout.contiguous(), cos, sin, H, KVH, hd, -sign), None, None, None, None, None, None


rope_qkv.register_autograd(_rope_backward, setup_context=_rope_setup)


# ----------------------------------------------------------------------------- FlashAttention on the packed projection
def _split(qkv, H, KVH, hd):
    B, T, _ = qkv.shape
    return (qkv[..., : H * hd].view(B, T, H, hd), qkv[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd),
            qkv[..., (H + KVH) * hd:].view(B, T, KVH, hd))


@torch.library.custom_op(f"{NS}::flash_attn_packed", mutates_args=(), device_types="cuda")
def flash_attn_packed(qkv: Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> tuple[Tensor, Tensor]:
    qkv = qkv.contiguous()
    B, T, _ = qkv.shape
    q, k, v = _split(qkv, n_heads, n_kv_heads, head_dim)
    o = torch.empty((B, T, n_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    lse = attention.fwd_raw(q, k, v, o, 1.0 / math.sqrt(head_dim))
    return o.view(B, T, n_heads * head_dim), lse


@flash_attn_packed.register_fake
def _(qkv, n_heads, n_kv_heads, head_dim):
    B, T, _ = qkv.shape
    return qkv.new_empty((B, T, n_heads * head_dim)), qkv.new_empty((B, n_heads, T), dtype=torch.float32)


@torch.library.custom_op(f"{NS}::flash_attn_packed_bwd", mutates_args=(), device_types="cuda")
def flash_attn_packed_bwd(do: Tensor, qkv: Tensor, o: Tensor, lse: Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> Tensor:
    qkv, do = qkv.contiguous(), do.contiguous()
    B, T, _ = qkv.shape
    q, k, v = _split(qkv, n_heads, n_kv_heads, head_dim)
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = _split(dqkv, n_heads, n_kv_heads, head_dim)
    attention.bwd_raw(q, k, v, o.view(B, T, n_heads, head_dim), lse, do.view(B, T, n_heads, head_dim), dq, dk, dv, 1.0 / math.sqrt(head_dim))
    return dqkv


@flash_attn_packed_bwd.register_fake
def _(do, qkv, o, lse, n_heads, n_kv_heads, head_dim):
    return torch.empty_like(qkv, memory_format=torch.contiguous_format)


def _fa_setup(ctx, inputs, output):
    qkv, H, KVH, hd = inputs
    o, lse = output
    ctx.save_for_backward(qkv, o, lse)
    ctx.meta = (H, KVH, hd)


def _fa_backward(ctx, do, _dlse):
    qkv, o, lse = ctx.saved_tensors
    return flash_attn_packed_bwd(do, qkv, o, lse, *ctx.meta), None, None, None


flash_attn_packed.register_autograd(_fa_backward, setup_context=_fa_setup)


# ----------------------------------------------------------------------------- linear (tcgen05 GEMM), 16-bit weight
@torch.library.custom_op(f"{NS}::matmul_nt", mutates_args=(), device_types="cuda")
def matmul_nt(a: Tensor, b: Tensor, a_mn: bool = False, b_mn: bool = False, out_f32: bool = False) -> Tensor:
    """a @ b^T with the operand layouts of csrc/gemm.cu (a_mn / b_mn: the operand is stored transposed)."""
    return gemm_mod.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32 if out_f32 else None)


@matmul_nt.register_fake
def _(a, b, a_mn=False, b_mn=False, out_f32=False):
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    return a.new_empty((M, N), dtype=torch.float32 if out_f32 else a.dtype)


def _mm_setup(ctx, inputs, output):
    a, b, a_mn, b_mn, out_f32 = inputs
    assert not a_mn and not b_mn, "autograd is defined for the plain a @ b^T form"
    ctx.save_for_backward(a, b)


def _mm_backward(ctx, dy):
    a, b = ctx.saved_tensors
    dy = dy.to(a.dtype).contiguous()
    da = matmul_nt(dy, b, False, True, False)          # dy @ b
    db = matmul_nt(dy, a, True, True, False)           # dy^T @ a
    return da, db, None, None, None


matmul_nt.register_autograd(_mm_backward, setup_context=_mm_setup)


def linear(x: Tensor, w16: Tensor) -> Tensor:
    """x [..., K] @ w16 [N, K]^T through the registered operator."""
    return matmul_nt(x.reshape(-1, x.shape[-1]), w16).view(*x.shape[:-1], w16.shape[0])
