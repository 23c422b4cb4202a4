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


def _fused_call(name: str, *args) -> bool:
    """Launch a GEMM with a fused epilogue; False when the CTA-pair kernel does not serve the shape (the caller then runs
    the plain GEMM followed by the stand-alone elementwise kernel)."""
    return _lib.call_rc(name, *args) == 0


def gemm_swiglu(x2: torch.Tensor, w_gu: torch.Tensor):
    """x2 [M, K] @ w_gu [2F, K]^T with the SwiGLU activation in the epilogue -> (gu [M, 2F], act [M, F]) or None."""
    M, K = x2.shape
    F = w_gu.shape[0] // 2
    if M < 256 or F % 128 or w_gu.stride(1) != 1 or x2.stride(1) != 1:
        return None
    gu = torch.empty((M, 2 * F), dtype=x2.dtype, device=x2.device)
    act = torch.empty((M, F), dtype=x2.dtype, device=x2.device)
    ok = _fused_call("nnb_gemm_swiglu", _lib.ptr(x2), _lib.ptr(w_gu), _lib.ptr(gu), _lib.ptr(act), _lib.i32(M), _lib.i32(F),
                     _lib.i32(K), _lib.i64(x2.stride(0)), _lib.i64(w_gu.stride(0)), _lib.i64(2 * F), _lib.i64(F),
                     _lib.i32(_CODE[x2.dtype]), _lib.ptr(status_tensor(x2.device)), _lib.vp(_lib.stream_ptr()))
    return (gu, act) if ok else None


def gemm_swiglu_bwd(dy2: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor):
    """SwiGLU backward inside the down projection's input-gradient GEMM: dy2 [M, d] @ w_down [d, F] is the gradient of
    act = silu(gate) * up; the epilogue reads the saved projection gu [M, 2F] and writes d(gate) | d(up) [M, 2F] directly
    (the gradient of act is never stored) -> dgu or None when the CTA-pair kernel does not serve the shape."""
    M, K = dy2.shape
    F = w_down.shape[1]
    if (M < 256 or F < 128 or F % 64 or gu.shape != (M, 2 * F) or gu.stride(1) != 1 or gu.stride(0) % 8 or w_down.stride(1) != 1
            or dy2.stride(1) != 1 or gu.dtype != dy2.dtype or w_down.dtype != dy2.dtype):
        return None
    dgu = torch.empty((M, 2 * F), dtype=gu.dtype, device=gu.device)
    ok = _fused_call("nnb_gemm_swiglu_bwd", _lib.ptr(dy2), _lib.ptr(w_down), _lib.ptr(gu), _lib.ptr(dgu), _lib.i32(M), _lib.i32(F),
                     _lib.i32(K), _lib.i64(dy2.stride(0)), _lib.i64(w_down.stride(0)), _lib.i64(gu.stride(0)), _lib.i64(2 * F),
                     _lib.i32(_CODE[dy2.dtype]), _lib.ptr(status_tensor(dy2.device)), _lib.vp(_lib.stream_ptr()))
    return dgu if ok else None


def gemm_rope(x2: torch.Tensor, w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, t_len: int, rope_cols: int, head_dim: int):
    """x2 [M, K] @ w [N, K]^T with rotate-half RoPE on columns [0, rope_cols) in the epilogue (row m at position
    m % t_len; cos / sin fp32 [t_len, head_dim / 2] contiguous) -> [M, N] or None."""
    M, K = x2.shape
    N = w.shape[0]
    if M < 256 or N < 128 or head_dim not in (64, 128) or N % head_dim or rope_cols % head_dim:
        return None
    out = torch.empty((M, N), dtype=x2.dtype, device=x2.device)
    ok = _fused_call("nnb_gemm_rope", _lib.ptr(x2), _lib.ptr(w), _lib.ptr(out), _lib.ptr(cos), _lib.ptr(sin), _lib.i32(M), _lib.i32(N),
                     _lib.i32(K), _lib.i64(x2.stride(0)), _lib.i64(w.stride(0)), _lib.i64(N), _lib.i32(t_len), _lib.i32(rope_cols),
                     _lib.i32(head_dim), _lib.i32(_CODE[x2.dtype]), _lib.ptr(status_tensor(x2.device)), _lib.vp(_lib.stream_ptr()))
    return out if ok else None


def gemm_ce_stats(x2: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """out [M, N] = x2 @ w^T plus partial softmax statistics (max, sum of exp(x - max)) of every row, two parts per
    256-column tile -> stats fp32 [M, 2 ceil(N / 256), 2] or None."""
    M, K = x2.shape
    N = w.shape[0]
    if M < 256 or N < 128 or N % 64:
        return None
    stats = torch.empty((M, 2 * ((N + 255) // 256), 2), dtype=torch.float32, device=x2.device)
    ok = _fused_call("nnb_gemm_ce_stats", _lib.ptr(x2), _lib.ptr(w), _lib.ptr(out), _lib.ptr(stats), _lib.i32(M), _lib.i32(N),
                     _lib.i32(K), _lib.i64(x2.stride(0)), _lib.i64(w.stride(0)), _lib.i64(out.stride(0)), _lib.i32(_CODE[x2.dtype]),
                     _lib.ptr(status_tensor(x2.device)), _lib.vp(_lib.stream_ptr()))
    return stats if ok else None


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
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx, dw = linear_backward(dy2, x2, weight, ctx.w16, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if dx is not None:
            dx = dx.view(*dy.shape[:-1], x2.shape[-1])
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, dw


def linear_backward(dy2, x2, weight, w16, need_dx: bool, need_dw: bool):
    """The two backward GEMMs of ``y = x2 @ w16^T``: returns (dx [M, K] or None, dW for autograd or None).
    When the weight has a slot in the flat gradient buffer (``weight._main_grad``) the weight gradient is accumulated
    there in fp32 by the GEMM epilogue, the strategy is told the gradient is complete (``_grad_ready_cb``) and the
    returned dW is None."""
    if dy2.dtype != x2.dtype:
        dy2 = dy2.to(x2.dtype)
    dy2 = _rowmajor2d(dy2)
    dx = dw = None
    if need_dx:
        dx = gemm(dy2, w16, b_mn=True)  # [M, K_in]
    if need_dw:
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


# ----------------------------------------------------------------------------- GEMMs fused with a collective
class FusedCollectiveGemm:
    """Per-group state for the two single-kernel compute+collective GEMMs (csrc/gemm.cu modes 1 and 2):
    the symmetric flag buffer, the local flag words, the epoch counter and the status words.

    ``gemm_rs(a, b, out)``  row-parallel linear: every rank multiplies its K-slice for ALL rows and each
    output tile is TMA-reduce-added over NVLink into the rank that owns those rows (``out`` is a
    ``SymmetricBuffer`` holding this rank's [M / world, N] shard).
    ``ag_gemm(a_full, b)``  column-parallel linear: ``a_full`` is a ``SymmetricBuffer`` of the FULL
    [M, K] activation in which each rank has written only its own row range; a few CTAs pull the peers'
    ranges in while the rest multiply, starting with the local rows.
    """

    def __init__(self, device, group, rank: int, world: int, max_m_blocks: int = 4096, gather_ctas: int = 16):
        from nanonemo_b200.parallel.symm import SymmetricBuffer

        self.rank, self.world, self.group, self.gather_ctas = rank, world, group, gather_ctas
        words = _lib.lib().nnb_comm_flag_words(max(1, gather_ctas))
        self.flags = SymmetricBuffer(words, torch.int32, device, group)
        self.flags.tensor.zero_()
        self.local_flags = torch.zeros(2 + max_m_blocks, dtype=torch.int32, device=device)
        self.comm_status = torch.zeros(8, dtype=torch.int32, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        torch.distributed.barrier(group)

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, out, *, b_mn: bool = False, out_f32: bool = False):
        """a: [M, K_local]; b: [N, K_local] (or [K_local, N] when b_mn); out: SymmetricBuffer viewed as
        [M / world, N]. Returns this rank's reduced shard (valid once the kernel has run)."""
        a, b = _rowmajor2d(a), _rowmajor2d(b)
        M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        shard = out.tensor.view(-1)[: (M // self.world) * N].view(M // self.world, N)
        shard.zero_()
        self.epoch += 1
        _lib.call("nnb_gemm_rs_bf16", _lib.ptr(a), _lib.ptr(b), out.ptr_array, self.flags.ptr_array, _lib.ptr(self.local_flags),
                  _lib.ptr(self.comm_status), _lib.i32(self.rank), _lib.i32(self.world), _lib.i32(self.epoch), _lib.i32(M),
                  _lib.i32(N), _lib.i32(K), _lib.i64(a.stride(0)), _lib.i64(b.stride(0)), _lib.i64(N), _lib.i32(int(b_mn)),
                  _lib.i32(_CODE[a.dtype]), _lib.i32(int(out_f32)), _lib.ptr(status_tensor(a.device)), _lib.vp(_lib.stream_ptr()))
        return shard

    def ag_gemm(self, a_full, M: int, K: int, b: torch.Tensor, *, b_mn: bool = False, out: torch.Tensor | None = None):
        """a_full: SymmetricBuffer holding [M, K] 16-bit with this rank's rows already written."""
        b = _rowmajor2d(b)
        N = b.shape[1] if b_mn else b.shape[0]
        dtype = a_full.tensor.dtype
        out = out if out is not None else torch.empty((M, N), dtype=dtype, device=b.device)
        self.epoch += 1
        _lib.call("nnb_ag_gemm_bf16", a_full.ptr_array, _lib.ptr(b), _lib.ptr(out), self.flags.ptr_array, _lib.ptr(self.local_flags),
                  _lib.ptr(self.comm_status), _lib.i32(self.rank), _lib.i32(self.world), _lib.i32(self.epoch),
                  _lib.i32(self.gather_ctas), _lib.i32(M), _lib.i32(N), _lib.i32(K), _lib.i64(b.stride(0)), _lib.i64(out.stride(0)),
                  _lib.i32(int(b_mn)), _lib.i32(_CODE[dtype]), _lib.ptr(status_tensor(b.device)), _lib.vp(_lib.stream_ptr()))
        return out

    def gather_b_gemm(self, a: torch.Tensor, wire, src_off_bytes: int, per_bytes: int, unit_dst: torch.Tensor, b_off_bytes: int,
                      N: int, out: torch.Tensor | None = None):
        """a [M, K] @ B[N, K]^T where B sits `b_off_bytes` into a parameter unit sharded over the ranks (`wire`:
        SymmetricBuffer with every rank's shard at `src_off_bytes`, `per_bytes` each). The kernel all-gathers the WHOLE unit
        into `unit_dst` (this rank's unsharded 16-bit copy) while it multiplies: afterwards every parameter of the unit is local."""
        a = _rowmajor2d(a)
        M, K = a.shape
        out = out if out is not None else torch.empty((M, N), dtype=a.dtype, device=a.device)
        chunks = self.world * ((per_bytes + 32767) // 32768)
        assert 2 + chunks <= self.local_flags.numel(), "unit too large for the flag table"
        self.epoch += 1
        _lib.call("nnb_gather_b_gemm_bf16", _lib.ptr(a), wire.ptr_array, _lib.ptr(unit_dst), _lib.ptr(out), self.flags.ptr_array,
                  _lib.ptr(self.local_flags), _lib.ptr(self.comm_status), _lib.i32(self.rank), _lib.i32(self.world), _lib.i32(self.epoch),
                  _lib.i32(self.gather_ctas), _lib.i64(src_off_bytes), _lib.i64(per_bytes), _lib.i64(b_off_bytes), _lib.i32(M), _lib.i32(N),
                  _lib.i32(K), _lib.i64(a.stride(0)), _lib.i64(out.stride(0)), _lib.i32(_CODE[a.dtype]), _lib.ptr(status_tensor(a.device)),
                  _lib.vp(_lib.stream_ptr()))
        return out

    def check_status(self):
        st = self.comm_status.tolist()
        if st[0] != 0:
            self.comm_status.zero_()
            raise RuntimeError(f"fused GEMM collective gave up waiting: code={st[0]} rank={st[1]} peer={st[2]} block={st[3]} epoch={st[4]}")
        check_status()
