"""tcgen05 GEMM front end (csrc/gemm.cu) and the ``linear`` built on it.

``gemm(a, b, ...)`` computes ``D[M, N] (+)= A[M, K] @ B[N, K]^T`` for 16-bit inputs with fp32
accumulation. Each operand can be given K-major (as ``[rows, K]``) or MN-major (the transposed
storage ``[K, rows]``), which is what lets the three GEMMs of a linear layer run without a
transposed copy of the weight or of any activation:

    fprop  y  = x @ W^T       a = x  [M, K]            b = W  [N, K]
    dgrad  dx = dy @ W        a = dy [M, N_out]        b = W  [N_out, K_in] read as B^T (MN-major)
    wgrad  dW += dy^T @ x     a = dy read as A^T, b = x read as B^T, fp32 out, split-K, reduce-add

``linear_sm100(x, weight)`` is the autograd function: the weight is the fp32 master parameter; the
16-bit copy it multiplies with is ``weight._shadow`` (maintained by the flat parameter store and
rewritten by the fused AdamW kernel) or a cast made on the fly; the weight gradient is accumulated
in fp32 directly into the flat gradient buffer when there is one.
"""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.bfloat16: 1, torch.float16: 2}
_status: dict = {}


def status_tensor(device) -> torch.Tensor:
    key = (device.type, device.index)
    t = _status.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device=None):
    """Raise if any GEMM launched so far on `device` gave up on a bounded wait (synchronises)."""
    for key, t in _status.items():
        code, role, block, item = t.tolist()
        if code != 0:
            t.zero_()
            raise RuntimeError(f"tcgen05 GEMM gave up waiting: role={role} (1 producer, 2 mma, 3 epilogue) block={block} item={item}")


def _rowmajor2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, accumulate: bool = False, k_splits: int = 0, bn: int = 0,
         max_ctas: int = 0) -> torch.Tensor:
    """a: [M, K] (or [K, M] when a_mn); b: [N, K] (or [K, N] when b_mn) -> out [M, N]."""
    a, b = _rowmajor2d(a), _rowmajor2d(b)
    assert a.dtype == b.dtype and a.dtype in _CODE, f"gemm needs matching bf16/fp16 inputs, got {a.dtype}/{b.dtype}"
    K, M = (a.shape if a_mn else a.shape[::-1])
    Kb, N = (b.shape if b_mn else b.shape[::-1])
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    assert out_dtype in (a.dtype, torch.float32)
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype == out_dtype
    _lib.call("nnb_gemm_bf16", _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.i32(M), _lib.i32(N), _lib.i32(K),
              _lib.i64(a.stride(0)), _lib.i64(b.stride(0)), _lib.i64(out.stride(0)), _lib.i32(int(a_mn)), _lib.i32(int(b_mn)),
              _lib.i32(_CODE[a.dtype]), _lib.i32(int(out_dtype == torch.float32)), _lib.i32(int(accumulate)),
              _lib.i32(k_splits), _lib.i32(bn), _lib.i32(max_ctas), _lib.ptr(status_tensor(a.device)),
              _lib.vp(_lib.stream_ptr()))
    return out


def compute_dtype() -> torch.dtype:
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        if dt in _CODE:
            return dt
    return torch.bfloat16


def shadow_of(weight: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    sh = getattr(weight, "_shadow", None)
    if sh is not None and sh.dtype == dtype:
        return sh
    return weight.detach().to(dtype)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        dt = compute_dtype()
        w16 = shadow_of(weight, dt)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != dt:
            x2 = x2.to(dt)
        x2 = _rowmajor2d(x2)
        y = gemm(x2, w16)
        ctx.save_for_backward(x2, weight)
        ctx.w16 = w16
        ctx.x_dtype = x.dtype
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        w16 = ctx.w16
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != x2.dtype:
            dy2 = dy2.to(x2.dtype)
        dy2 = _rowmajor2d(dy2)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w16, b_mn=True)  # [M, K_in]
            dx = dx.view(*dy.shape[:-1], x2.shape[-1])
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "_main_grad", None)
            if main is not None and main.dtype == torch.float32:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
                cb = getattr(weight, "_grad_ready_cb", None)
                if cb is not None and not getattr(weight, "_tied_embedding", False):
                    cb(weight, True)  # a tied head weight is complete only after the embedding backward
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(weight.dtype)
        return dx, dw


def linear_sm100(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _Linear.apply(x, weight)
