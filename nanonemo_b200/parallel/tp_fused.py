"""Tensor-parallel linears whose collective is INSIDE the GEMM kernel (csrc/gemm.cu modes 1 and 2).

Column-parallel (``wqkv``, ``w_gu``): forward is all-gather -> GEMM in one kernel (the activation
shards are pulled from the peers' symmetric buffers while the local rows are already being
multiplied); the input gradient is GEMM -> reduce-scatter in one kernel (every output tile is
reduce-added over NVLink into the rank that owns those token rows).
Row-parallel (``wo``, ``w_down``): forward is GEMM -> reduce-scatter, the input gradient is
all-gather -> GEMM. Weight gradients are local GEMMs on the gathered operand, accumulated in fp32
straight into the flat gradient buffer.

These replace the DTensor ``PrepareModuleInput`` / ``ColwiseParallel`` / ``RowwiseParallel`` pairs of
the reference (nanonemo/distributed/tp.py:52-64), which issue separate NCCL collectives around cuBLAS.
"""

import torch

from nanonemo_b200.ops.gemm import FusedCollectiveGemm, compute_dtype, gemm, shadow_of
from nanonemo_b200.parallel.symm import SymmetricBuffer, SymmetricComm


class FusedTP:
    """Symmetric staging buffers + the fused-GEMM launcher for one tensor-parallel group."""

    def __init__(self, device, group, rank, world, max_tokens: int, max_width: int, dtype=torch.bfloat16):
        self.rank, self.world, self.dtype = rank, world, dtype
        self.fg = FusedCollectiveGemm(device, group, rank, world, max_m_blocks=max(4096, max_tokens // 128))
        # full-size gather source/destination (tokens x widest gathered operand) and reduce-scatter target
        self.gather_buf = SymmetricBuffer(max_tokens * max_width, dtype, device, group)
        self.shard_buf = SymmetricBuffer((max_tokens // world) * max_width, dtype, device, group)
        # vocabulary-parallel embedding: a light-kernel communicator and a staging area for this rank's rows (fp32 at most)
        self.comm = SymmetricComm(device, group, rank, world)
        self.embed_stage = SymmetricBuffer((max_tokens // world) * max_width, torch.float32, device, group)

    def gathered_matmul(self, x_shard, w, b_mn=False):
        """all-gather(x_shard over token rows) @ w^T in one kernel. Returns (y [M, N], x_full view).
        The view stays valid until the next gathered_matmul."""
        Ms, K = x_shard.shape
        M = Ms * self.world
        full = self.gather_buf.tensor.view(-1)[: M * K].view(M, K)
        full[self.rank * Ms:(self.rank + 1) * Ms].copy_(x_shard)
        y = self.fg.ag_gemm(self.gather_buf, M, K, w, b_mn=b_mn)
        return y, full

    def matmul_scattered(self, a, w, b_mn=False):
        """reduce-scatter(a @ w^T over token rows) in one kernel -> this rank's [M / world, N] rows."""
        return self.fg.gemm_rs(a, w, self.shard_buf, b_mn=b_mn).clone()


    def embed_rows(self, idx_flat, weight, v0: int, out_dtype):
        """This rank's token rows of the vocabulary-sharded table: every rank pushes the rows it owns to the token owners."""
        per = idx_flat.numel() // self.world
        out = torch.empty((per, weight.shape[1]), dtype=out_dtype, device=weight.device)
        self.comm.vp_embedding(self.embed_stage, idx_flat, out, weight, v0, backward=False)
        return out

    def embed_grad(self, idx_flat, g, table_grad, v0: int):
        """table_grad[idx - v0] += gradient rows of the tokens whose id falls in this rank's slice, pulled from their owners."""
        self.comm.vp_embedding(self.embed_stage, idx_flat, g, table_grad, v0, backward=True)


class _ColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, tp):
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        xs = x_shard if x_shard.dtype == dt else x_shard.to(dt)
        y, x_full = tp.gathered_matmul(xs.contiguous(), w16)
        ctx.save_for_backward(x_full.clone(), weight)  # the gather buffer is reused by the next layer
        ctx.tp, ctx.w16, ctx.x_dtype = tp, w16, x_shard.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight = ctx.saved_tensors
        tp, w16 = ctx.tp, ctx.w16
        dy = dy.contiguous() if dy.dtype == w16.dtype else dy.to(w16.dtype).contiguous()
        dx = tp.matmul_scattered(dy, w16, b_mn=True).to(ctx.x_dtype)  # [M / tp, K]: partial sums reduced in the epilogue
        main = getattr(weight, "_main_grad", None)
        dw = None
        if main is not None and main.dtype == torch.float32:
            gemm(dy, x_full, a_mn=True, b_mn=True, out=main, accumulate=True)
            cb = getattr(weight, "_grad_ready_cb", None)
            if cb is not None:
                cb(weight, True)
        else:
            dw = gemm(dy, x_full, a_mn=True, b_mn=True, out_dtype=torch.float32).to(weight.dtype)
        return dx, dw, None


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_full, weight, tp):
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        x = x_full if x_full.dtype == dt else x_full.to(dt)
        x = x.contiguous()
        y_shard = tp.matmul_scattered(x, w16)
        ctx.save_for_backward(x, weight)
        ctx.tp, ctx.w16, ctx.x_dtype = tp, w16, x_full.dtype
        return y_shard

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        tp, w16 = ctx.tp, ctx.w16
        dys = dy_shard.contiguous() if dy_shard.dtype == w16.dtype else dy_shard.to(w16.dtype).contiguous()
        dx, dy_full = tp.gathered_matmul(dys, w16, b_mn=True)  # [M, K_local]
        main = getattr(weight, "_main_grad", None)
        dw = None
        if main is not None and main.dtype == torch.float32:
            gemm(dy_full, x, a_mn=True, b_mn=True, out=main, accumulate=True)
            cb = getattr(weight, "_grad_ready_cb", None)
            if cb is not None:
                cb(weight, True)
        else:
            dw = gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(weight.dtype)
        return dx.to(ctx.x_dtype), dw, None


def column_parallel_linear(x_shard, weight, tp: FusedTP):
    """x_shard [M / tp, K] (this rank's tokens) -> [M, N_local]."""
    return _ColumnParallel.apply(x_shard, weight, tp)


def row_parallel_linear(x_full, weight, tp: FusedTP):
    """x_full [M, K_local] -> this rank's [M / tp, N] rows of the summed product."""
    return _RowParallel.apply(x_full, weight, tp)
