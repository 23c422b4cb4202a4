"""Fused linear + cross-entropy over the tied LM head: mean CE of ``x @ W^T`` without the logits.

Row chunks of the flattened hidden states go through: logits chunk (tcgen05 GEMM, bf16, whose epilogue
also reduces every 256-column tile of a row to its (max, sum-exp)) -> one-sweep in-place CE kernel (combines the tile
statistics, writes the loss per row, overwrites the logits with ``(softmax - onehot) / N``) -> ``dx`` chunk
and ``dW +=`` (tcgen05 GEMMs, the latter accumulating in fp32). As in the reference operator
(nanonemo/kernels/triton/linear_ce.py:44-80) the gradients are produced during the forward pass and
backward only rescales them by the upstream gradient; the chunk is sized for B200 (32768 rows: one
chunk's 16-bit logits are 3.3 GB of the 180 GB, and the three GEMMs fill all 148 SMs for several
waves; the reference uses 512-row chunks on 8 GB parts).
"""

import torch

from nanonemo_b200.ops import _lib
from nanonemo_b200.ops.gemm import _CODE, compute_dtype, gemm, gemm_ce_stats, shadow_of

DEFAULT_CHUNK_ROWS = 32768


def ce_inplace(logits: torch.Tensor, targets: torch.Tensor, loss_rows: torch.Tensor, grad_scale: float):
    R, V = logits.shape
    _lib.call("nnb_ce_inplace", _lib.ptr(logits), _lib.ptr(targets), _lib.ptr(loss_rows), _lib.i64(R), _lib.i32(V),
              _lib.i64(logits.stride(0)), _lib.f32(grad_scale), _lib.i32(_CODE[logits.dtype]), _lib.vp(_lib.stream_ptr()))


def ce_from_stats(logits: torch.Tensor, targets: torch.Tensor, tile_stats: torch.Tensor, loss_rows: torch.Tensor, grad_scale: float):
    """One-sweep form of `ce_inplace`: `tile_stats` [R, n_tiles, 2] came out of the head GEMM's epilogue (gemm_ce_stats)."""
    R, V = logits.shape
    _lib.call("nnb_ce_grad_from_stats", _lib.ptr(logits), _lib.ptr(targets), _lib.ptr(tile_stats), _lib.i32(tile_stats.shape[1]),
              _lib.ptr(loss_rows), _lib.i64(R), _lib.i32(V), _lib.i64(logits.stride(0)), _lib.f32(grad_scale),
              _lib.i32(_CODE[logits.dtype]), _lib.vp(_lib.stream_ptr()))


FUSE_STATS = True  # head GEMM epilogue produces the softmax statistics (tests switch it off to compare the two routes)


def linear_ce_fwd(x16, w16, targets, chunk_rows, dW_out):
    """Returns (sum of row losses [fp32 scalar], dx [N, D] 16-bit for the MEAN loss); accumulates the
    mean-loss weight gradient into dW_out (fp32 [V, D])."""
    N, D = x16.shape
    V = w16.shape[0]
    chunk_rows = min(chunk_rows, N)
    dx = torch.empty_like(x16)
    loss_rows = torch.empty(N, dtype=torch.float32, device=x16.device)
    logits = torch.empty((chunk_rows, V), dtype=x16.dtype, device=x16.device)
    for r0 in range(0, N, chunk_rows):
        r1 = min(r0 + chunk_rows, N)
        lg = logits[: r1 - r0]
        xc = x16[r0:r1]
        stats = gemm_ce_stats(xc, w16, lg) if FUSE_STATS else None
        if stats is not None:
            ce_from_stats(lg, targets[r0:r1], stats, loss_rows[r0:r1], 1.0 / N)
        else:
            gemm(xc, w16, out=lg)
            ce_inplace(lg, targets[r0:r1], loss_rows[r0:r1], 1.0 / N)
        gemm(lg, w16, b_mn=True, out=dx[r0:r1], bn=0 if r1 - r0 >= 16384 else 128)
        gemm(lg, xc, a_mn=True, b_mn=True, out=dW_out, accumulate=True)
    return loss_rows.sum(), dx


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, targets, chunk_rows):
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        x16 = x if x.dtype == dt else x.to(dt)
        x16 = x16 if x16.is_contiguous() else x16.contiguous()
        tg = targets if targets.dtype == torch.int64 else targets.long()
        tg = tg if tg.is_contiguous() else tg.contiguous()
        need_grad = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)
        dW = torch.zeros(weight.shape, dtype=torch.float32, device=x.device)
        loss_sum, dx = linear_ce_fwd(x16, w16, tg, chunk_rows or DEFAULT_CHUNK_ROWS, dW)
        ctx.save_for_backward(dx, dW, weight)
        ctx.x_dtype = x.dtype
        return loss_sum / x.shape[0]

    @staticmethod
    def backward(ctx, dloss):
        dx, dW, weight = ctx.saved_tensors
        gx = (dx * dloss.to(dx.dtype)).to(ctx.x_dtype) if ctx.needs_input_grad[0] else None
        gw = None
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "_main_grad", None)
            if main is not None and main.dtype == torch.float32:
                main.addcmul_(dW, dloss)  # readiness of the tied weight is reported by the embedding backward
            else:
                gw = (dW * dloss).to(weight.dtype)
        return gx, gw, None, None


def linear_cross_entropy(x, weight, targets, chunk_rows=None):
    """x: [N, D]; weight: [V, D] (fp32 master or 16-bit); targets: [N] int64 -> scalar mean loss (fp32)."""
    return _LinearCE.apply(x, weight, targets, chunk_rows)


# ----------------------------------------------------------------------------- vocabulary-parallel variant
def _ce_stats(logits, targets, stats, v0):
    R, V = logits.shape
    _lib.call("nnb_ce_stats", _lib.ptr(logits), _lib.ptr(targets), _lib.ptr(stats), _lib.i64(R), _lib.i32(V),
              _lib.i64(logits.stride(0)), _lib.i64(v0), _lib.i32(_CODE[logits.dtype]), _lib.vp(_lib.stream_ptr()))


def _ce_grad_vp(logits, targets, stats_all, loss_rows, v0, v_total, world, grad_scale):
    R, V = logits.shape
    _lib.call("nnb_ce_grad_vp", _lib.ptr(logits), _lib.ptr(targets), _lib.ptr(stats_all), _lib.ptr(loss_rows), _lib.i64(R),
              _lib.i32(V), _lib.i64(logits.stride(0)), _lib.i64(v0), _lib.i64(v_total), _lib.i32(world), _lib.f32(grad_scale),
              _lib.i32(_CODE[logits.dtype]), _lib.vp(_lib.stream_ptr()))


def vocab_parallel_ce_inplace(logits, targets, loss_rows, grad_scale, v0, v_total, all_gather, world):
    """Cross entropy over vocabulary shards, in place: `logits` is this rank's [R, V/world] slice (columns v0..), targets are
    global ids. One launch reduces the slice to (max, sum-exp, target logit) per row, `all_gather` (callable: [R, 4] fp32 ->
    [world * R, 4]) exchanges those 16 bytes per row, and a second launch combines them, writes the row losses and overwrites
    the slice with (softmax - onehot) * grad_scale. Full logits are never gathered and no fp32 copy of the slice is made."""
    stats = torch.empty((logits.shape[0], 4), dtype=torch.float32, device=logits.device)
    _ce_stats(logits, targets, stats, v0)
    stats_all = all_gather(stats) if world > 1 else stats
    _ce_grad_vp(logits, targets, stats_all, loss_rows, v0, v_total, world, grad_scale)


class _VocabParallelLinearCE(torch.autograd.Function):
    """Fused linear + cross entropy with the head sharded over the vocabulary: x [N, D] (all tokens), weight [V/world, D].
    The returned dx is this rank's PARTIAL sum over its vocabulary slice (the caller's token gather reduce-scatters it)."""

    @staticmethod
    def forward(ctx, x, weight, targets, tp, v0, chunk_rows):
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        x16 = x if x.dtype == dt else x.to(dt)
        x16 = x16 if x16.is_contiguous() else x16.contiguous()
        tg = (targets if targets.dtype == torch.int64 else targets.long()).contiguous()
        N, D = x16.shape
        Vl = w16.shape[0]
        rows = min(chunk_rows or DEFAULT_CHUNK_ROWS, N)
        dx = torch.empty_like(x16)
        dW = torch.zeros(weight.shape, dtype=torch.float32, device=x.device)
        loss_rows = torch.empty(N, dtype=torch.float32, device=x.device)
        logits = torch.empty((rows, Vl), dtype=dt, device=x.device)
        for r0 in range(0, N, rows):
            r1 = min(r0 + rows, N)
            lg, xc = logits[: r1 - r0], x16[r0:r1]
            gemm(xc, w16, out=lg)
            vocab_parallel_ce_inplace(lg, tg[r0:r1], loss_rows[r0:r1], 1.0 / N, v0, Vl * tp.world, tp.all_gather, tp.world)
            gemm(lg, w16, b_mn=True, out=dx[r0:r1], bn=0 if r1 - r0 >= 16384 else 128)
            gemm(lg, xc, a_mn=True, b_mn=True, out=dW, accumulate=True)
        ctx.save_for_backward(dx, dW, weight)
        ctx.x_dtype = x.dtype
        return loss_rows.sum() / N

    @staticmethod
    def backward(ctx, dloss):
        dx, dW, weight = ctx.saved_tensors
        gx = (dx * dloss.to(dx.dtype)).to(ctx.x_dtype) if ctx.needs_input_grad[0] else None
        gw = None
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "_main_grad", None)
            if main is not None and main.dtype == torch.float32:
                main.add_(dW * dloss)  # readiness of the tied weight is reported by the embedding backward
            else:
                gw = (dW * dloss).to(weight.dtype)
        return gx, gw, None, None, None, None


def vocab_parallel_linear_cross_entropy(x, weight_local, targets, tp, v0, chunk_rows=None):
    """x: [N, D] (every token); weight_local: [V/tp, D] rows v0.. of the head; targets: [N] global ids -> scalar mean loss."""
    return _VocabParallelLinearCE.apply(x, weight_local, targets, tp, v0, chunk_rows)
