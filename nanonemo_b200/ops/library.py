"""``torch.library`` registration of the sm100 operators: schema + fake (meta) implementation + autograd formula
for each, so they compose with ``torch.compile(fullgraph=True)``, ``opcheck`` and functional transforms — the binding
layer of the reference (nanonemo/kernels/cuda/rmsnorm.py:1-69, flash_attn.py:1-60: ``custom_op`` + ``register_fake`` +
``register_autograd``), on top of the ahead-of-time built library instead of a per-process JIT.

These operators ARE the model's sm100 path: ``nanonemo_b200.ops`` routes every call here unless the parameter involved
lives in a flat parameter store (``weight._main_grad``), where the trainer's variants accumulate weight gradients in
place in the flat buffer and report gradient readiness to the strategy — side effects a functional operator cannot
have. Both routes call the same launchers.

    torch.ops.nanonemo_b200.add_rms_norm(x, delta, weight, eps)              -> (y, h, rstd)
    torch.ops.nanonemo_b200.swiglu(gu)                                       -> act
    torch.ops.nanonemo_b200.rope_qkv(qkv, cos, sin, H, KVH, hd, sign)        -> qkv_rot
    torch.ops.nanonemo_b200.flash_attn_packed(qkv, H, KVH, hd)               -> (o, lse)
    torch.ops.nanonemo_b200.matmul_nt(a, b, a_mn, b_mn, out_f32)             -> a @ b^T
    torch.ops.nanonemo_b200.linear_w(x2, weight)                             -> x2 @ weight^T (fp32 or 16-bit weight)
    torch.ops.nanonemo_b200.gemm_rope(x2, weight, cos, sin, T, cols, hd)     -> projection with RoPE in the epilogue
    torch.ops.nanonemo_b200.gemm_swiglu(x2, weight)                          -> (gu, act) with SwiGLU in the epilogue
    torch.ops.nanonemo_b200.embedding(idx, weight, fp32_out)                 -> rows
    torch.ops.nanonemo_b200.linear_ce(x2, weight, targets, chunk_rows)       -> (mean loss, dx, dW)
    torch.ops.nanonemo_b200.adamw_step(p, g, m, v, shadow, flags, ...)       -> None (mutates its buffers)
"""

import math

import torch
from torch import Tensor

from nanonemo_b200.ops import adamw as adamw_mod, attention, embed as embed_mod, gemm as gemm_mod, linear_ce as ce_mod, rmsnorm, rope, swiglu_act

NS = "nanonemo_b200"


# ----------------------------------------------------------------------------- add + RMSNorm
_DT = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}
_DT_CODE = {v: k for k, v in _DT.items()}


@torch.library.custom_op(f"{NS}::add_rms_norm", mutates_args=(), device_types="cuda")
def add_rms_norm(x: Tensor, delta: Tensor | None, weight: Tensor, eps: float, y_code: int = -1) -> tuple[Tensor, Tensor, Tensor]:
    """(y, h, rstd): h = x + delta (x itself without a delta), y = rmsnorm(h) * weight in dtype code y_code (0 fp32, 1 bf16,
    2 fp16; -1 = the delta's dtype, or x's without a delta)."""
    y_dtype = _DT[y_code] if y_code >= 0 else (delta.dtype if delta is not None else x.dtype)
    y, h, rstd = rmsnorm.fwd(x, delta, weight, eps, y_dtype)
    return y, (h if delta is not None else h.clone()), rstd


@add_rms_norm.register_fake
def _(x, delta, weight, eps, y_code=-1):
    y_dtype = _DT[y_code] if y_code >= 0 else (delta.dtype if delta is not None else x.dtype)
    return (x.new_empty(x.shape, dtype=y_dtype), torch.empty_like(x, memory_format=torch.contiguous_format),
            x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32))


@torch.library.custom_op(f"{NS}::add_rms_norm_bwd", mutates_args=(), device_types="cuda")
def add_rms_norm_bwd(dy: Tensor, dh: Tensor | None, h: Tensor, rstd: Tensor, weight: Tensor, delta_code: int) -> tuple[Tensor, Tensor, Tensor]:
    """(dx, ddelta, dw); ddelta has dtype code delta_code (when it equals the residual dtype it is a copy of dx)."""
    dx, ddelta, dw = rmsnorm.bwd(dy, h, rstd, weight, dh, _DT[delta_code])
    return dx, ddelta if ddelta is not dx else dx.clone(), dw


@add_rms_norm_bwd.register_fake
def _(dy, dh, h, rstd, weight, delta_code):
    return torch.empty_like(h), h.new_empty(h.shape, dtype=_DT[delta_code]), weight.new_empty(weight.shape, dtype=torch.float32)


def _arn_setup(ctx, inputs, output):
    x, delta, weight, _, _ = inputs
    y, h, rstd = output
    ctx.save_for_backward(h, rstd, weight)
    ctx.has_delta = delta is not None
    ctx.delta_code = _DT_CODE[delta.dtype if delta is not None else y.dtype]
    ctx.y_dtype = y.dtype
    ctx.set_materialize_grads(False)


def _arn_backward(ctx, dy, dh, _drstd):
    h, rstd, weight = ctx.saved_tensors
    dy = dy.contiguous() if dy is not None else torch.zeros(h.shape, dtype=ctx.y_dtype, device=h.device)
    dx, ddelta, dw = add_rms_norm_bwd(dy, dh.contiguous() if dh is not None else None, h, rstd, weight, ctx.delta_code)
    return dx, (ddelta if ctx.has_delta else None), dw.to(weight.dtype), None, None


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




# ----------------------------------------------------------------------------- linear with the weight as given (fp32 master or 16-bit)
def _w16(weight: Tensor, dtype: torch.dtype) -> Tensor:
    return weight if weight.dtype == dtype else weight.to(dtype)


@torch.library.custom_op(f"{NS}::linear_w", mutates_args=(), device_types="cuda")
def linear_w(x2: Tensor, weight: Tensor) -> Tensor:
    """x2 [M, K] (16-bit) @ weight [N, K]^T; an fp32 weight is cast to x2's dtype for the product."""
    return gemm_mod.gemm(x2, _w16(weight, x2.dtype))


@linear_w.register_fake
def _(x2, weight):
    return x2.new_empty((x2.shape[0], weight.shape[0]))


def _linw_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _linw_backward(ctx, dy):
    x2, weight = ctx.saved_tensors
    dy = dy.to(x2.dtype).contiguous()
    dx = matmul_nt(dy, _w16(weight, x2.dtype), False, True, False)
    dw = matmul_nt(dy, x2, True, True, True)  # fp32 accumulate and output: the master weight's gradient keeps full precision
    return dx, dw.to(weight.dtype)


linear_w.register_autograd(_linw_backward, setup_context=_linw_setup)


def linear(x: Tensor, weight: Tensor) -> Tensor:
    """x [..., K] @ weight [N, K]^T in the autocast dtype (bf16 by default) through the registered operator."""
    dt = gemm_mod.compute_dtype()
    x2 = x.reshape(-1, x.shape[-1])
    x2 = x2 if x2.dtype == dt else x2.to(dt)
    return linear_w(x2.contiguous(), weight).view(*x.shape[:-1], weight.shape[0])


# ----------------------------------------------------------------------------- RoPE on 2-D rows (any column count, in / out of place)
@torch.library.custom_op(f"{NS}::rope_rows", mutates_args=(), device_types="cuda")
def rope_rows(x2: Tensor, cos: Tensor, sin: Tensor, t_len: int, n_rot_heads: int, head_dim: int, sign: float) -> Tensor:
    """Rotate-half on the first n_rot_heads heads of every row (row m at position m % t_len), other columns copied."""
    x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
    out = torch.empty(x2.shape, dtype=x2.dtype, device=x2.device)
    rope.rope_packed_raw(x2, out, cos, sin, t_len, n_rot_heads, head_dim, x2.shape[1] - n_rot_heads * head_dim, sign)
    return out


@rope_rows.register_fake
def _(x2, cos, sin, t_len, n_rot_heads, head_dim, sign):
    return torch.empty_like(x2, memory_format=torch.contiguous_format)


def _rr_setup(ctx, inputs, output):
    _, cos, sin, t_len, n_rot, hd, sign = inputs
    ctx.save_for_backward(cos, sin)
    ctx.meta = (t_len, n_rot, hd, sign)


def _rr_backward(ctx, dout):
    cos, sin = ctx.saved_tensors
    t_len, n_rot, hd, sign = ctx.meta
    return rope_rows(dout.contiguous(), cos, sin, t_len, n_rot, hd, -sign), None, None, None, None, None, None


rope_rows.register_autograd(_rr_backward, setup_context=_rr_setup)


# ----------------------------------------------------------------------------- GEMMs with a fused epilogue
@torch.library.custom_op(f"{NS}::gemm_rope", mutates_args=(), device_types="cuda")
def gemm_rope(x2: Tensor, weight: Tensor, cos: Tensor, sin: Tensor, t_len: int, rope_cols: int, head_dim: int) -> Tensor:
    """x2 @ weight^T with RoPE on columns [0, rope_cols) in the GEMM epilogue (plain GEMM + RoPE kernel for shapes the
    fused kernel does not serve: same result)."""
    w16 = _w16(weight, x2.dtype)
    out = gemm_mod.gemm_rope(x2, w16, cos, sin, t_len, rope_cols, head_dim)
    if out is None:
        out = gemm_mod.gemm(x2, w16)
        rope.rope_packed_raw(out, out, cos, sin, t_len, rope_cols // head_dim, head_dim, 0, 1.0)
    return out


@gemm_rope.register_fake
def _(x2, weight, cos, sin, t_len, rope_cols, head_dim):
    return x2.new_empty((x2.shape[0], weight.shape[0]))


def _gr_setup(ctx, inputs, output):
    x2, weight, cos, sin, t_len, rope_cols, hd = inputs
    ctx.save_for_backward(x2, weight, cos, sin)
    ctx.meta = (t_len, rope_cols, hd)


def _gr_backward(ctx, dout):
    x2, weight, cos, sin = ctx.saved_tensors
    t_len, rope_cols, hd = ctx.meta
    draw = rope_rows(dout.to(x2.dtype).contiguous(), cos, sin, t_len, rope_cols // hd, hd, -1.0)
    dx = matmul_nt(draw, _w16(weight, x2.dtype), False, True, False)
    dw = matmul_nt(draw, x2, True, True, True)
    return dx, dw.to(weight.dtype), None, None, None, None, None


gemm_rope.register_autograd(_gr_backward, setup_context=_gr_setup)


@torch.library.custom_op(f"{NS}::gemm_swiglu", mutates_args=(), device_types="cuda")
def gemm_swiglu(x2: Tensor, weight: Tensor) -> tuple[Tensor, Tensor]:
    """(gu, act): gu = x2 @ weight^T with gate columns first, act = silu(gate) * up written by the GEMM epilogue."""
    w16 = _w16(weight, x2.dtype)
    fused = gemm_mod.gemm_swiglu(x2, w16)
    if fused is not None:
        return fused
    gu = gemm_mod.gemm(x2, w16)
    F = gu.shape[1] // 2
    act = torch.empty((gu.shape[0], F), dtype=gu.dtype, device=gu.device)
    swiglu_act.fwd_raw(gu[:, :F], gu[:, F:], act)
    return gu, act


@gemm_swiglu.register_fake
def _(x2, weight):
    return x2.new_empty((x2.shape[0], weight.shape[0])), x2.new_empty((x2.shape[0], weight.shape[0] // 2))


def _gs_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs, output[0])


def _gs_backward(ctx, dgu, dact):
    x2, weight, gu = ctx.saved_tensors
    total = None
    if dact is not None:
        total = swiglu_bwd(dact.to(gu.dtype).contiguous(), gu)
    if dgu is not None:
        total = dgu.to(gu.dtype) if total is None else total + dgu.to(gu.dtype)
    total = total.contiguous()
    dx = matmul_nt(total, _w16(weight, x2.dtype), False, True, False)
    dw = matmul_nt(total, x2, True, True, True)
    return dx, dw.to(weight.dtype)


gemm_swiglu.register_autograd(_gs_backward, setup_context=_gs_setup)


# ----------------------------------------------------------------------------- embedding
@torch.library.custom_op(f"{NS}::embedding", mutates_args=(), device_types="cuda")
def embedding(idx: Tensor, weight: Tensor, fp32_out: bool = True) -> Tensor:
    """weight[idx] from the fp32 table, written in fp32 or bf16 (the dtype of the residual stream)."""
    w = weight if weight.dtype == torch.float32 else weight.float()
    out, _ = embed_mod.fwd_raw(idx, w.contiguous(), torch.float32 if fp32_out else torch.bfloat16)
    return out


@embedding.register_fake
def _(idx, weight, fp32_out=True):
    return weight.new_empty((*idx.shape, weight.shape[1]), dtype=torch.float32 if fp32_out else torch.bfloat16)


@torch.library.custom_op(f"{NS}::embedding_bwd", mutates_args=(), device_types="cuda")
def embedding_bwd(idx: Tensor, dout: Tensor, vocab: int) -> Tensor:
    """fp32 [vocab, D] with dout's rows added at idx (rows that repeat are summed)."""
    flat = idx.reshape(-1)
    flat = (flat if flat.dtype == torch.int64 else flat.long()).contiguous()
    dW = torch.zeros((vocab, dout.shape[-1]), dtype=torch.float32, device=dout.device)
    embed_mod.bwd_raw(flat, dout.contiguous(), dW)
    return dW


@embedding_bwd.register_fake
def _(idx, dout, vocab):
    return dout.new_empty((vocab, dout.shape[-1]), dtype=torch.float32)


def _emb_setup(ctx, inputs, output):
    idx, weight, _ = inputs
    ctx.save_for_backward(idx)
    ctx.vocab, ctx.w_dtype = weight.shape[0], weight.dtype


def _emb_backward(ctx, dout):
    (idx,) = ctx.saved_tensors
    return None, embedding_bwd(idx, dout, ctx.vocab).to(ctx.w_dtype), None


embedding.register_autograd(_emb_backward, setup_context=_emb_setup)


# ----------------------------------------------------------------------------- fused linear + cross-entropy
@torch.library.custom_op(f"{NS}::linear_ce", mutates_args=(), device_types="cuda")
def linear_ce(x2: Tensor, weight: Tensor, targets: Tensor, chunk_rows: int) -> tuple[Tensor, Tensor, Tensor]:
    """Mean cross-entropy of x2 @ weight^T against targets, and the gradients of that mean with respect to x2 (16-bit)
    and weight (fp32), all produced in the same pass (the logits exist one row chunk at a time, in 16 bits)."""
    w16 = _w16(weight, x2.dtype)
    tg = (targets if targets.dtype == torch.int64 else targets.long()).contiguous()
    dW = torch.zeros(weight.shape, dtype=torch.float32, device=x2.device)
    loss_sum, dx = ce_mod.linear_ce_fwd(x2, w16.contiguous(), tg, chunk_rows, dW)
    return loss_sum / x2.shape[0], dx, dW


@linear_ce.register_fake
def _(x2, weight, targets, chunk_rows):
    return x2.new_empty((), dtype=torch.float32), torch.empty_like(x2), weight.new_empty(weight.shape, dtype=torch.float32)


def _lce_setup(ctx, inputs, output):
    ctx.save_for_backward(output[1], output[2])
    ctx.w_dtype = inputs[1].dtype
    ctx.set_materialize_grads(False)


def _lce_backward(ctx, dloss, _ddx, _ddw):
    dx, dW = ctx.saved_tensors
    if dloss is None:
        return None, None, None, None
    return dx * dloss.to(dx.dtype), (dW * dloss).to(ctx.w_dtype), None, None


linear_ce.register_autograd(_lce_backward, setup_context=_lce_setup)


def linear_cross_entropy(x: Tensor, weight: Tensor, targets: Tensor, chunk_rows: int | None = None) -> Tensor:
    """x: [N, D]; weight: [V, D] (fp32 master or 16-bit); targets: [N] -> scalar mean loss (fp32)."""
    dt = gemm_mod.compute_dtype()
    x2 = x if x.dtype == dt else x.to(dt)
    loss, _, _ = linear_ce(x2.contiguous(), weight, targets, chunk_rows or ce_mod.DEFAULT_CHUNK_ROWS)
    return loss


# ----------------------------------------------------------------------------- fused clip + AdamW on flat buffers
@torch.library.custom_op(f"{NS}::adamw_step", mutates_args=("p", "g", "m", "v", "shadow"), device_types="cuda")
def adamw_step(p: Tensor, g: Tensor, m: Tensor, v: Tensor, shadow: Tensor | None, decay_flags: Tensor, grad_norm_sq: Tensor | None,
               lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int, max_norm: float,
               zero_grad: bool) -> None:
    """One launch: clip by the global norm (grad_norm_sq on the device, max_norm <= 0 = no clipping), AdamW on the fp32
    master weights and moments, 16-bit shadow written, gradient zeroed. decay_flags: one byte per 256 elements."""
    adamw_mod.adamw_flat(p, g, m, v, shadow, decay_flags, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                         step=step, grad_norm_sq=grad_norm_sq if max_norm > 0 else None, max_norm=max_norm if max_norm > 0 else None,
                         zero_grad=zero_grad)


@adamw_step.register_fake
def _(p, g, m, v, shadow, decay_flags, grad_norm_sq, lr, beta1, beta2, eps, weight_decay, step, max_norm, zero_grad):
    return None


# ----------------------------------------------------------------------------- SwiGLU on separate gate / up tensors
@torch.library.custom_op(f"{NS}::swiglu_gu", mutates_args=(), device_types="cuda")
def swiglu_gu(g: Tensor, u: Tensor) -> Tensor:
    g2, u2 = swiglu_act._rows(g), swiglu_act._rows(u)
    out = torch.empty((g2.shape[0], g2.shape[1]), dtype=g.dtype, device=g.device)
    swiglu_act.fwd_raw(g2, u2, out)
    return out.view(g.shape)


@swiglu_gu.register_fake
def _(g, u):
    return torch.empty_like(g, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{NS}::swiglu_gu_bwd", mutates_args=(), device_types="cuda")
def swiglu_gu_bwd(dy: Tensor, g: Tensor, u: Tensor) -> tuple[Tensor, Tensor]:
    g2, u2, dy2 = swiglu_act._rows(g), swiglu_act._rows(u), swiglu_act._rows(dy)
    dg = torch.empty((g2.shape[0], g2.shape[1]), dtype=g.dtype, device=g.device)
    du = torch.empty_like(dg)
    swiglu_act.bwd_raw(dy2, g2, u2, dg, du)
    return dg.view(g.shape), du.view(g.shape)


@swiglu_gu_bwd.register_fake
def _(dy, g, u):
    return torch.empty_like(g, memory_format=torch.contiguous_format), torch.empty_like(g, memory_format=torch.contiguous_format)


swiglu_gu.register_autograd(lambda ctx, dy: swiglu_gu_bwd(dy.contiguous(), *ctx.saved_tensors),
                            setup_context=lambda ctx, inputs, output: ctx.save_for_backward(*inputs))


# ----------------------------------------------------------------------------- FlashAttention on separate (B, H, T, hd) tensors
def _bthd(t: Tensor) -> Tensor:
    """(B, heads, T, hd) -> the kernel's [B, T, heads, hd] view; copied only when strides / alignment rule it out."""
    t = t.transpose(1, 2)
    ok = t.stride(-1) == 1 and all((s * 2) % 16 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


@torch.library.custom_op(f"{NS}::flash_attn", mutates_args=(), device_types="cuda")
def flash_attn(q: Tensor, k: Tensor, v: Tensor) -> tuple[Tensor, Tensor]:
    """Causal GQA attention on bf16 q (B, H, T, hd), k / v (B, KVH, T, hd) -> (o (B, H, T, hd), lse (B, H, T))."""
    qt, kt, vt = _bthd(q), _bthd(k), _bthd(v)
    B, T, H, hd = qt.shape
    o = torch.empty((B, T, H, hd), dtype=q.dtype, device=q.device)
    lse = attention.fwd_raw(qt, kt, vt, o, 1.0 / math.sqrt(hd))
    return o.transpose(1, 2), lse


@flash_attn.register_fake
def _(q, k, v):
    B, H, T, hd = q.shape
    return q.new_empty((B, T, H, hd)).transpose(1, 2), q.new_empty((B, H, T), dtype=torch.float32)


@torch.library.custom_op(f"{NS}::flash_attn_bwd", mutates_args=(), device_types="cuda")
def flash_attn_bwd(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    qt, kt, vt, ot, dot = _bthd(q), _bthd(k), _bthd(v), _bthd(o), _bthd(do)
    hd = qt.shape[-1]
    dq = torch.empty(qt.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(kt.shape, dtype=q.dtype, device=q.device)
    dv = torch.empty(vt.shape, dtype=q.dtype, device=q.device)
    attention.bwd_raw(qt, kt, vt, ot, lse, dot, dq, dk, dv, 1.0 / math.sqrt(hd))
    return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)


@flash_attn_bwd.register_fake
def _(do, q, k, v, o, lse):
    mk = lambda t: t.new_empty((t.shape[0], t.shape[2], t.shape[1], t.shape[3])).transpose(1, 2)
    return mk(q), mk(k), mk(v)


def _fl_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs, *output)


def _fl_backward(ctx, do, _dlse):
    q, k, v, o, lse = ctx.saved_tensors
    return flash_attn_bwd(do.to(q.dtype), q, k, v, o, lse)


flash_attn.register_autograd(_fl_backward, setup_context=_fl_setup)
