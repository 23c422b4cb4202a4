"""Operator front end: one function per hot operator, each with a plain-PyTorch implementation
(``impl="torch"``: the oracle, and the only path on CPU) and the hand-written Blackwell kernel
(``impl="sm100"``) from ``nanonemo_b200/csrc``. There is no third backend and no runtime probing:
asking for ``sm100`` without the built library, or off a CUDA device, raises.

Operator contracts follow the reference kernels (nanonemo/kernels/triton/*.py,
nanonemo/kernels/cuda/*.py): ``add_rms_norm(x, delta, w, eps) -> (y, h)``, RoPE on Q and K in one
launch, ``swiglu``, ``flash_attn(q, k, v)`` reading KV heads directly, ``linear_cross_entropy``.
"""

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel


# ----------------------------------------------------------------------------- torch oracles
def rms_norm_torch(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * weight.float()).to(x.dtype)


def add_rms_norm_torch(x, delta, weight, eps):
    if delta is not None:
        x = x + delta
    return rms_norm_torch(x, weight, eps), x


def rope_torch(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_dim: int = -2) -> torch.Tensor:
    """Rotate-half RoPE in fp32. x: (..., T, hd) with seq_dim=-2, or (B, T, H, hd) with seq_dim=1."""
    half = x.shape[-1] // 2
    T = x.shape[seq_dim]
    cos, sin = cos[:T], sin[:T]
    if seq_dim in (1, -3):
        cos, sin = cos[:, None, :], sin[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    return torch.cat((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).to(x.dtype)


def attention_torch(q, k, v, backend=SDPBackend.MATH):
    """q: (B, H, T, hd); k, v: (B, KVH, T, hd). Query head h uses KV head h // (H // KVH)."""
    group = q.shape[1] // k.shape[1]
    if group > 1:
        k = k.repeat_interleave(group, dim=1)
        v = v.repeat_interleave(group, dim=1)
    with sdpa_kernel(backend):
        return F.scaled_dot_product_attention(q, k, v, is_causal=True)


def swiglu_torch(g, u):
    return F.silu(g) * u


def linear_cross_entropy_torch(x, weight, targets):
    return F.cross_entropy(F.linear(x, weight).float(), targets)


# ----------------------------------------------------------------------------- dispatch
def _need_cuda(t: torch.Tensor, op: str):
    if not t.is_cuda:
        raise RuntimeError(f"{op}: impl='sm100' needs a CUDA tensor (got {t.device}); use impl='torch' on CPU")


def linear(x, weight, impl="torch"):
    if impl == "torch":
        return F.linear(x, weight)
    _need_cuda(x, "linear")
    if impl == "mxfp8":
        from nanonemo_b200.fp8 import linear_mxfp8

        return linear_mxfp8(x, weight)
    from nanonemo_b200.ops.gemm import linear_sm100

    return linear_sm100(x, weight)


def add_rms_norm(x, delta, weight, eps, impl="torch"):
    if impl == "torch":
        return add_rms_norm_torch(x, delta, weight, eps)
    _need_cuda(x, "add_rms_norm")
    from nanonemo_b200.ops.rmsnorm import add_rms_norm as f

    return f(x, delta, weight, eps)


def rope_qkv(qkv, cos, sin, n_heads, n_kv_heads, head_dim, impl="torch"):
    """RoPE on the Q and K columns of a packed (B, T, (H + 2 KVH) hd) projection; V is passed through."""
    if impl == "torch":
        B, T, _ = qkv.shape
        qd, kd = n_heads * head_dim, n_kv_heads * head_dim
        q, k, v = qkv.split((qd, kd, kd), dim=-1)
        q = rope_torch(q.reshape(B, T, n_heads, head_dim), cos, sin, seq_dim=1).reshape(B, T, qd)
        k = rope_torch(k.reshape(B, T, n_kv_heads, head_dim), cos, sin, seq_dim=1).reshape(B, T, kd)
        return torch.cat((q, k, v), dim=-1)
    _need_cuda(qkv, "rope_qkv")
    from nanonemo_b200.ops.rope import rope_qkv as f

    return f(qkv, cos, sin, n_heads, n_kv_heads, head_dim)


def apply_rope_qk(q, k, cos, sin, impl="torch"):
    """RoPE on q (B, T, H, hd) and k (B, T, KVH, hd) in one call; returns contiguous tensors."""
    if impl == "torch":
        return rope_torch(q, cos, sin, seq_dim=1), rope_torch(k, cos, sin, seq_dim=1)
    _need_cuda(q, "apply_rope_qk")
    from nanonemo_b200.ops.rope import apply_rope_qk as f

    return f(q, k, cos, sin)


def attention_packed(qkv, n_heads, n_kv_heads, head_dim, impl="torch", backend=SDPBackend.MATH):
    """Causal GQA attention on a packed (B, T, (H + 2 KVH) hd) projection -> (B, T, H hd)."""
    B, T, _ = qkv.shape
    qd, kd = n_heads * head_dim, n_kv_heads * head_dim
    if impl == "torch":
        q, k, v = qkv.split((qd, kd, kd), dim=-1)
        q = q.view(B, T, n_heads, head_dim).transpose(1, 2)
        k = k.view(B, T, n_kv_heads, head_dim).transpose(1, 2)
        v = v.view(B, T, n_kv_heads, head_dim).transpose(1, 2)
        return attention_torch(q, k, v, backend).transpose(1, 2).reshape(B, T, qd)
    _need_cuda(qkv, "attention_packed")
    from nanonemo_b200.ops.attention import flash_attn_packed

    return flash_attn_packed(qkv, n_heads, n_kv_heads, head_dim)


def flash_attn(q, k, v, impl="sm100"):
    """q: (B, H, T, hd), k/v: (B, KVH, T, hd), any strides with a contiguous last dim -> (B, H, T, hd)."""
    if impl == "torch":
        return attention_torch(q, k, v)
    _need_cuda(q, "flash_attn")
    from nanonemo_b200.ops.attention import flash_attn as f

    return f(q, k, v)


def swiglu(g, u, impl="torch"):
    if impl == "torch":
        return swiglu_torch(g, u)
    _need_cuda(g, "swiglu")
    from nanonemo_b200.ops.swiglu_act import swiglu as f

    return f(g, u)


def swiglu_packed(gu, impl="torch"):
    """gu: (..., 2 F) with gate in the first F columns and up in the last F -> (..., F)."""
    if impl == "torch":
        g, u = gu.chunk(2, dim=-1)
        return swiglu_torch(g, u)
    _need_cuda(gu, "swiglu_packed")
    from nanonemo_b200.ops.swiglu_act import swiglu_packed as f

    return f(gu)


def fused_ok() -> bool:
    """The block-level fused operators compute in bf16 (the attention kernels are bf16 only)."""
    from nanonemo_b200.ops.gemm import compute_dtype

    return compute_dtype() == torch.bfloat16


def qkv_rope_attention(x, weight, cos, sin, n_heads, n_kv_heads, head_dim):
    """Packed QKV projection + RoPE (GEMM epilogue) + causal GQA attention as one autograd node (sm100 only)."""
    _need_cuda(x, "qkv_rope_attention")
    from nanonemo_b200.ops.fused_block import qkv_rope_attention as f

    return f(x, weight, cos, sin, n_heads, n_kv_heads, head_dim)


def linear_swiglu(x, weight):
    """gate||up projection with silu(gate) * up written by the GEMM epilogue (sm100 only)."""
    _need_cuda(x, "linear_swiglu")
    from nanonemo_b200.ops.fused_block import linear_swiglu as f

    return f(x, weight)


def embedding(idx, weight, impl="torch"):
    if impl == "torch":
        return F.embedding(idx, weight)
    _need_cuda(weight, "embedding")
    from nanonemo_b200.ops.embed import embedding as f

    return f(idx, weight)


def linear_cross_entropy(x, weight, targets, impl="sm100", chunk_rows=None):
    """Mean next-token cross entropy of ``x @ weight.T`` without materialising the full logits."""
    if impl == "torch" or not x.is_cuda:
        return linear_cross_entropy_torch(x, weight, targets)
    from nanonemo_b200.ops.linear_ce import linear_cross_entropy as f

    return f(x, weight, targets, chunk_rows)
