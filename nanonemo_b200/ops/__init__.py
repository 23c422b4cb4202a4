"""Operator front end: one function per hot operator, each with a plain-PyTorch implementation
(``impl="torch"``: the oracle, and the only path on CPU) and the hand-written Blackwell kernel
(``impl="sm100"``) from ``nanonemo_b200/csrc``. There is no third backend and no runtime probing:
asking for ``sm100`` without the built library, or off a CUDA device, raises.

The sm100 kernels are bound once, as ``torch.library`` custom operators with fake implementations and autograd
formulas (``ops/library.py``), and that is what these functions call. The exception is the trainer's engine: a
parameter that lives in a flat parameter store (it carries ``_main_grad``) runs its operators as ``autograd.Function``s
that accumulate the weight gradient in place in the flat fp32 buffer and tell the strategy when it is complete — what a
functional operator may not do — and once such a store exists the weightless operators take the direct functions of
``ops/direct.py`` too (no dispatcher round trip on the hot path). Both routes launch the same kernels.

Operator contracts follow the reference kernels (nanonemo/kernels/triton/*.py,
nanonemo/kernels/cuda/*.py): ``add_rms_norm(x, delta, w, eps) -> (y, h)``, RoPE on Q and K in one
launch, ``swiglu``, ``flash_attn(q, k, v)`` reading KV heads directly, ``linear_cross_entropy``.
"""

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

_ATTN_DTYPES = (torch.bfloat16, torch.float16)  # operand formats of the tensor-core attention kernels


# ----------------------------------------------------------------------------- torch oracles
def _wide(x: torch.Tensor) -> torch.Tensor:
    """The dtype the oracles do their arithmetic in: fp32, or fp64 for fp64 inputs (gradcheck)."""
    return x if x.dtype == torch.float64 else x.float()


def rms_norm_torch(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = _wide(x)
    xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * weight.to(xf.dtype)).to(x.dtype)


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
    xf = _wide(x)
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
    return F.cross_entropy(_wide(F.linear(x, weight)), targets)


# ----------------------------------------------------------------------------- dispatch
def _need_cuda(t: torch.Tensor, op: str):
    if not t.is_cuda:
        raise RuntimeError(f"{op}: impl='sm100' needs a CUDA tensor (got {t.device}); use impl='torch' on CPU")


def in_flat_store(weight) -> bool:
    """True for a parameter of the trainer's flat store: its gradient is accumulated in place by the backward kernels."""
    return getattr(weight, "_main_grad", None) is not None


def linear(x, weight, impl="torch"):
    if impl == "torch":
        return F.linear(x, weight)
    _need_cuda(x, "linear")
    if impl == "mxfp8":
        from nanonemo_b200.fp8 import linear_mxfp8

        return linear_mxfp8(x, weight)
    if in_flat_store(weight) or getattr(weight, "_shadow", None) is not None:
        from nanonemo_b200.ops.gemm import linear_sm100

        return linear_sm100(x, weight)
    from nanonemo_b200.ops import library

    return library.linear(x, weight)


def add_rms_norm(x, delta, weight, eps, impl="torch"):
    if impl == "torch":
        return add_rms_norm_torch(x, delta, weight, eps)
    _need_cuda(x, "add_rms_norm")
    from nanonemo_b200.ops import rmsnorm

    if in_flat_store(weight):
        return rmsnorm.add_rms_norm(x, delta, weight, eps)
    from nanonemo_b200.ops import library

    y_dtype = rmsnorm._y_dtype(x, delta)
    if delta is not None and delta.dtype != y_dtype:
        delta = delta.to(y_dtype)
    if x.dtype not in (torch.float32, y_dtype):
        x = x.float()
    y, h, _ = library.add_rms_norm(x, delta, weight, eps, library._DT_CODE[y_dtype])
    return y, h


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
    from nanonemo_b200.ops import direct, library
    from nanonemo_b200.ops.rope import _tables

    c, s = _tables(cos, sin, qkv.shape[1])
    if direct.ENABLED:
        return direct.rope_qkv(qkv, c, s, n_heads, n_kv_heads, head_dim)
    return library.rope_qkv(qkv, c, s, n_heads, n_kv_heads, head_dim)


def apply_rope_qk(q, k, cos, sin, impl="torch"):
    """RoPE on q (B, T, H, hd) and k (B, T, KVH, hd) in one call; returns contiguous tensors."""
    if impl == "torch":
        return rope_torch(q, cos, sin, seq_dim=1), rope_torch(k, cos, sin, seq_dim=1)
    _need_cuda(q, "apply_rope_qk")
    from nanonemo_b200.ops import library
    from nanonemo_b200.ops.rope import _tables

    B, T, H, hd = q.shape
    KVH = k.shape[2]
    c, s = _tables(cos, sin, T)
    packed = torch.cat((q.reshape(B * T, H * hd), k.reshape(B * T, KVH * hd)), dim=-1)
    out = library.rope_rows(packed, c, s, T, H + KVH, hd, 1.0)
    return out[:, :H * hd].reshape(B, T, H, hd), out[:, H * hd:].reshape(B, T, KVH, hd)


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
    from nanonemo_b200.ops import direct, library

    if qkv.dtype not in _ATTN_DTYPES:  # the attention kernels take 16-bit operands: fp32 inputs go through bf16 and back
        return attention_packed(qkv.to(torch.bfloat16), n_heads, n_kv_heads, head_dim, impl, backend).to(qkv.dtype)
    if direct.ENABLED:
        return direct.flash_attn_packed(qkv, n_heads, n_kv_heads, head_dim)
    return library.flash_attn_packed(qkv, n_heads, n_kv_heads, head_dim)[0]


def flash_attn(q, k, v, impl="sm100"):
    """q: (B, H, T, hd), k/v: (B, KVH, T, hd), any strides with a contiguous last dim -> (B, H, T, hd)."""
    if impl == "torch":
        return attention_torch(q, k, v)
    _need_cuda(q, "flash_attn")
    from nanonemo_b200.ops import library

    dt = q.dtype if q.dtype in _ATTN_DTYPES else torch.bfloat16  # 16-bit operands of one dtype; fp32 goes through bf16 and back
    return library.flash_attn(q.to(dt), k.to(dt), v.to(dt))[0].to(q.dtype)


def swiglu(g, u, impl="torch"):
    if impl == "torch":
        return swiglu_torch(g, u)
    _need_cuda(g, "swiglu")
    from nanonemo_b200.ops import library

    return library.swiglu_gu(g, u if u.dtype == g.dtype else u.to(g.dtype))


def swiglu_packed(gu, impl="torch"):
    """gu: (..., 2 F) with gate in the first F columns and up in the last F -> (..., F)."""
    if impl == "torch":
        g, u = gu.chunk(2, dim=-1)
        return swiglu_torch(g, u)
    _need_cuda(gu, "swiglu_packed")
    from nanonemo_b200.ops import direct, library

    return direct.swiglu_packed(gu) if direct.ENABLED else library.swiglu(gu)


def fused_ok() -> bool:
    """The block-level fused operators run when the compute dtype is one the tensor-core kernels take (bf16 or fp16)."""
    from nanonemo_b200.ops.gemm import compute_dtype

    return compute_dtype() in _ATTN_DTYPES


def qkv_rope_attention(x, weight, cos, sin, n_heads, n_kv_heads, head_dim):
    """Packed QKV projection + RoPE (GEMM epilogue) + causal GQA attention (sm100 only)."""
    _need_cuda(x, "qkv_rope_attention")
    if in_flat_store(weight) or getattr(weight, "_shadow", None) is not None:
        from nanonemo_b200.ops.fused_block import qkv_rope_attention as f

        return f(x, weight, cos, sin, n_heads, n_kv_heads, head_dim)  # one autograd node, inverse RoPE inside the attention backward
    from nanonemo_b200.ops import library
    from nanonemo_b200.ops.rope import _tables

    B, T, _ = x.shape
    c, s = _tables(cos, sin, T)
    from nanonemo_b200.ops.gemm import compute_dtype

    x2 = x.reshape(B * T, -1).to(compute_dtype()).contiguous()
    qkv = library.gemm_rope(x2, weight, c, s, T, (n_heads + n_kv_heads) * head_dim, head_dim).view(B, T, -1)
    return library.flash_attn_packed(qkv, n_heads, n_kv_heads, head_dim)[0]


def linear_swiglu(x, weight):
    """gate||up projection with silu(gate) * up written by the GEMM epilogue (sm100 only)."""
    _need_cuda(x, "linear_swiglu")
    if in_flat_store(weight) or getattr(weight, "_shadow", None) is not None:
        from nanonemo_b200.ops.fused_block import linear_swiglu as f

        return f(x, weight)
    from nanonemo_b200.ops import library

    from nanonemo_b200.ops.gemm import compute_dtype

    x2 = x.reshape(-1, x.shape[-1]).to(compute_dtype()).contiguous()
    return library.gemm_swiglu(x2, weight)[1].view(*x.shape[:-1], weight.shape[0] // 2)


def mlp_swiglu(x, w_gu, w_down):
    """The SwiGLU feed-forward down(silu(gate(x)) * up(x)) (sm100 only). On the trainer's engine (weights with a 16-bit
    shadow) it is one autograd node whose backward computes the activation's backward in a GEMM epilogue; elsewhere it is
    the registered gate||up operator followed by the registered linear."""
    _need_cuda(x, "mlp_swiglu")
    engine = lambda w: in_flat_store(w) or getattr(w, "_shadow", None) is not None
    if engine(w_gu) and engine(w_down) and getattr(w_gu, "_gather_in_gemm", None) is None:
        from nanonemo_b200.ops.fused_block import mlp_swiglu as f

        return f(x, w_gu, w_down)
    return linear(linear_swiglu(x, w_gu), w_down, impl="sm100")


def embedding(idx, weight, impl="torch"):
    if impl == "torch":
        return F.embedding(idx, weight)
    _need_cuda(weight, "embedding")
    if in_flat_store(weight):
        from nanonemo_b200.ops.embed import embedding as f

        return f(idx, weight)
    from nanonemo_b200.ops import library

    return library.embedding(idx, weight, True)


def linear_cross_entropy(x, weight, targets, impl="sm100", chunk_rows=None):
    """Mean next-token cross entropy of ``x @ weight.T`` without materialising the full logits."""
    if impl == "torch" or not x.is_cuda:
        return linear_cross_entropy_torch(x, weight, targets)
    if in_flat_store(weight) or getattr(weight, "_shadow", None) is not None:
        from nanonemo_b200.ops.linear_ce import linear_cross_entropy as f

        return f(x, weight, targets, chunk_rows)
    from nanonemo_b200.ops import library

    return library.linear_cross_entropy(x, weight, targets, chunk_rows)
