"""Transformer building blocks: RMSNorm, fused-add RMSNorm, RoPE, GQA attention, SwiGLU MLP, Block.

Mirrors the behaviour of the reference layers (nanonemo/model/layers.py:21-161) with two
structural differences chosen for the Blackwell GEMM path:

* the Q, K and V projections are one parameter ``wqkv`` of shape ``[(H + 2*KVH) * hd, d]`` and the
  gate and up projections one parameter ``w_gu`` of shape ``[2 * d_ff, d]``, so each is a single
  wide GEMM (N = 1280 and N = 4096 at the 114M shape) instead of three / two narrow ones;
* every operator goes through ``nanonemo_b200.ops``; the ``impl`` string picked by the config is
  either ``torch`` (plain PyTorch, the oracle and the CPU path) or ``sm100`` (hand-written CUDA).

``split_qkv`` / ``split_gu`` give the per-projection views for export to the reference / HF layout.
"""

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn.attention import SDPBackend, sdpa_kernel

from nanonemo_b200 import ops
from nanonemo_b200.models.config import ModelConfig


class Linear(nn.Module):
    """Bias-free linear layer. ``impl`` = torch (F.linear / cuBLAS) | sm100 (tcgen05 GEMM) | mxfp8."""

    def __init__(self, in_features: int, out_features: int, impl: str = "torch"):
        super().__init__()
        self.in_features, self.out_features, self.impl = in_features, out_features, impl
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        nn.init.normal_(self.weight, std=0.02)  # the model re-initialises every weight in reset_parameters()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, impl=self.impl)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, impl={self.impl}"


def make_linear(cfg: ModelConfig, in_features: int, out_features: int) -> Linear:
    return Linear(in_features, out_features, cfg.resolved().linear_impl)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm_torch(x, self.weight, self.eps)


class AddRMSNorm(RMSNorm):
    """forward(x, delta) -> (rmsnorm(x + delta), x + delta); delta=None normalises x alone.

    The residual stream travels as (x, delta) so the pending add and the norm are one pass over
    memory (reference contract: nanonemo/model/layers.py:34-52).
    """

    def __init__(self, dim: int, eps: float = 1e-5, impl: str = "torch"):
        super().__init__(dim, eps)
        self.impl = impl

    def forward(self, x, delta=None):
        return ops.add_rms_norm(x, delta, self.weight, self.eps, impl=self.impl)


def rope_cache(head_dim: int, max_seq_len: int, base: float = 10000.0, device=None):
    """cos/sin tables of shape (max_seq_len, head_dim // 2) in fp32; angle[m, i] = m * base^(-2i/hd)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    pos = torch.arange(max_seq_len, device=device, dtype=torch.float32)
    angles = torch.outer(pos, inv_freq)
    return angles.cos(), angles.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on x of shape (B, H, T, hd): pairs dimension i with i + hd/2, fp32 math."""
    return ops.rope_torch(x, cos, sin, seq_dim=-2)


class Attention(nn.Module):
    """Causal grouped-query attention: n_heads query heads share n_kv_heads K/V heads."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        r = cfg.resolved()
        self.n_heads, self.n_kv_heads, self.head_dim = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        self.q_dim, self.kv_dim = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        self.backend = {"math": SDPBackend.MATH, "mem_efficient": SDPBackend.EFFICIENT_ATTENTION}[cfg.attn_backend]
        self.wqkv = make_linear(cfg, cfg.d_model, self.q_dim + 2 * self.kv_dim)
        self.wo = make_linear(cfg, self.q_dim, cfg.d_model)
        self.rope_impl, self.attn_impl = r.rope_kernel, r.attn_kernel
        # one autograd node for projection + RoPE (GEMM epilogue) + attention when all three run on the sm100 kernels
        self.fused = cfg.fuse_epilogues and r.linear_impl == "sm100" and self.rope_impl == "sm100" and self.attn_impl == "sm100"
        self.tp = None  # parallel.tp.TPContext once the model has been sharded

    def split_qkv(self):
        """(wq, wk, wv) views of the fused projection weight."""
        return self.wqkv.weight.split((self.q_dim, self.kv_dim, self.kv_dim), dim=0)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            # sequence parallel: x holds 1/tp of the tokens; gather them, attend over the local heads,
            # and reduce-scatter the row-parallel projection's partial sums back to token shards
            if self.tp.fused_tp is not None and self.tp.pair == 1:
                from nanonemo_b200.parallel.tp_fused import column_parallel_linear, row_parallel_linear

                ft = self.tp.fused_tp  # the gather and the scatter happen inside the two GEMM kernels
                qkv = column_parallel_linear(x, self.wqkv.weight, ft).view(self.tp.B, self.tp.T, -1)
                y = self._attend(None, cos, sin, qkv=qkv, project=False)
                return row_parallel_linear(y.reshape(-1, y.shape[-1]), self.wo.weight, ft)
            full = self.tp.gather_tokens(x).view(self.tp.B, self.tp.T, -1)
            if self.tp.pair > 1:
                # two ranks share this head group and split its query rows: the first attends over (and projects) the first
                # half of every sequence, the second attends over the whole sequence and projects the second half; the rows
                # a rank does not own enter the reduce-scatter as zeros
                half = self.tp.T // 2
                if self.tp.pair_pos == 0:
                    mine = self._attend(full[:, :half], cos, sin)
                    out = torch.cat((mine, mine.new_zeros(self.tp.B, self.tp.T - half, mine.shape[-1])), dim=1)
                else:
                    mine = self.wo(self._attend(full, cos, sin, project=False)[:, half:])
                    out = torch.cat((mine.new_zeros(self.tp.B, half, mine.shape[-1]), mine), dim=1)
                return self.tp.scatter_tokens(out.reshape(-1, x.shape[-1]))
            return self.tp.scatter_tokens(self._attend(full, cos, sin).reshape(-1, x.shape[-1]))
        return self._attend(x, cos, sin)

    def _attend(self, x, cos, sin, qkv=None, project=True):
        H, KVH, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if qkv is None and self.fused and x.is_cuda and ops.fused_ok():
            y = ops.qkv_rope_attention(x, self.wqkv.weight, cos, sin, H, KVH, hd)
            return self.wo(y) if project else y
        if qkv is None:
            qkv = self.wqkv(x)  # (B, T, (H + 2 KVH) hd)
        B, T, _ = qkv.shape
        if self.rope_impl == "sm100" or self.attn_impl == "sm100":
            # Packed path: RoPE rewrites the Q and K columns of the packed projection in one
            # launch, attention reads Q/K/V heads from it through strides and each query head
            # reads its own KV head directly (no repeat_interleave, no transposes).
            qkv = ops.rope_qkv(qkv, cos, sin, H, KVH, hd, impl=self.rope_impl)
            y = ops.attention_packed(qkv, H, KVH, hd, impl=self.attn_impl, backend=self.backend)
            return self.wo(y) if project else y
        q, k, v = qkv.split((self.q_dim, self.kv_dim, self.kv_dim), dim=-1)
        q = apply_rope(q.view(B, T, H, hd).transpose(1, 2), cos, sin)
        k = apply_rope(k.view(B, T, KVH, hd).transpose(1, 2), cos, sin)
        v = v.view(B, T, KVH, hd).transpose(1, 2)
        y = ops.attention_torch(q, k, v, self.backend).transpose(1, 2).reshape(B, T, -1)  # (B, T, H hd)
        return self.wo(y) if project else y


def silu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    return F.silu(g) * u


class MLP(nn.Module):
    """SwiGLU feed-forward: down(silu(gate(x)) * up(x)) with gate and up as one GEMM."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        r = cfg.resolved()
        self.d_ff = cfg.d_ff
        self.w_gu = make_linear(cfg, cfg.d_model, 2 * cfg.d_ff)  # rows [0, d_ff) = gate, [d_ff, 2 d_ff) = up
        self.w_down = make_linear(cfg, cfg.d_ff, cfg.d_model)
        self.act_impl = r.swiglu_kernel
        self.fused = cfg.fuse_epilogues and r.linear_impl == "sm100" and self.act_impl == "sm100"
        self.tp = None

    def split_gu(self):
        return self.w_gu.weight.split((self.d_ff, self.d_ff), dim=0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            if self.tp.fused_tp is not None:
                from nanonemo_b200.parallel.tp_fused import column_parallel_linear, row_parallel_linear

                ft = self.tp.fused_tp
                act = ops.swiglu_packed(column_parallel_linear(x, self.w_gu.weight, ft), impl=self.act_impl)
                return row_parallel_linear(act, self.w_down.weight, ft)
            full = self.tp.gather_tokens(x)
            return self.tp.scatter_tokens(self.w_down(ops.swiglu_packed(self.w_gu(full), impl=self.act_impl)))
        if self.fused and x.is_cuda and ops.fused_ok():
            return ops.mlp_swiglu(x, self.w_gu.weight, self.w_down.weight)
        return self.w_down(ops.swiglu_packed(self.w_gu(x), impl=self.act_impl))


class Block(nn.Module):
    """Pre-norm block. Input (x, delta) with delta the previous sublayer output not yet added to x;
    output (x', delta') in the same convention (reference: nanonemo/model/layers.py:141-161)."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        impl = cfg.resolved().norm_kernel
        self.norm_attn = AddRMSNorm(cfg.d_model, cfg.norm_eps, impl)
        self.attn = Attention(cfg)
        self.norm_mlp = AddRMSNorm(cfg.d_model, cfg.norm_eps, impl)
        self.mlp = MLP(cfg)

    def forward(self, x, cos, sin, delta=None):
        h, x = self.norm_attn(x, delta)
        h, x = self.norm_mlp(x, self.attn(h, cos, sin))
        return x, self.mlp(h)
