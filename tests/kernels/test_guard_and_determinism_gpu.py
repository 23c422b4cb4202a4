"""Race and out-of-bounds detection without a sanitizer: guard bands around every output (sentinel-filled memory before and
after, checked bit for bit after the launch), NaN-poisoned outputs (an unwritten tile stays NaN), and run-twice bitwise
determinism for the kernels whose reduction order is fixed (anything that races on an mbarrier or a flag shows up as a
difference between two runs). Kernels that accumulate through fp32 reduce-adds in a free order (split-K GEMMs, dQ) are
checked with a tolerance elsewhere."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = -1.2345e30


def guarded(rows, cols, dtype, pad_rows=3, pad_cols=8):
    """A [rows, cols] view in the middle of a sentinel-filled buffer; cols are padded so the view's row stride is 16-byte aligned."""
    big = torch.full((rows + 2 * pad_rows, cols + 2 * pad_cols), SENTINEL, dtype=dtype, device=DEV)
    view = big[pad_rows:pad_rows + rows, pad_cols:pad_cols + cols]
    view.fill_(float("nan"))
    return big, view


def assert_guards_intact(big, view, pad_rows=3, pad_cols=8):
    ref = torch.full_like(big, SENTINEL)
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[pad_rows:pad_rows + view.shape[0], pad_cols:pad_cols + view.shape[1]] = False
    assert torch.equal(big[mask], ref[mask]), "a kernel wrote outside its output"
    assert not torch.isnan(view.float()).any(), "a kernel left part of its output unwritten"


@pytest.mark.parametrize("bn", [0, 256, 128, 512])
@pytest.mark.parametrize("M,N,K", [(304, 520, 136), (128, 128, 64), (1000, 776, 264), (2560, 264, 72)])
def test_gemm_writes_its_output_and_nothing_else(M, N, K, bn):
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(0)
    a, b = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(N, K, device=DEV).bfloat16()
    big, out = guarded(M, N, torch.bfloat16)
    gemm(a, b, out=out, bn=bn)
    check_status()
    assert_guards_intact(big, out)
    big32, out32 = guarded(M, N, torch.float32)
    out32.zero_()
    gemm(a.t().contiguous(), b.t().contiguous(), a_mn=True, b_mn=True, out=out32, accumulate=True, bn=bn)  # split-K reduce-adds
    check_status()
    assert_guards_intact(big32, out32)
    torch.testing.assert_close(out32, a.float() @ b.float().t(), rtol=2e-2, atol=2e-1)


def test_mxfp8_gemm_writes_its_output_and_nothing_else():
    from nanonemo_b200 import fp8
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(1)
    aq, asf, _, _ = fp8.quantize_mx(torch.randn(384, 256, device=DEV).bfloat16())
    bq, bsf, _, _ = fp8.quantize_mx(torch.randn(640, 256, device=DEV).bfloat16())
    big, out = guarded(384, 640, torch.bfloat16)
    fp8.gemm_mxfp8(aq, asf, bq, bsf, out=out)
    check_status()
    assert_guards_intact(big, out)


@pytest.mark.parametrize("B,H,KVH,T,hd", [(2, 4, 2, 200, 64), (1, 2, 1, 333, 128)])
def test_attention_outputs_are_fully_written_and_nothing_else(B, H, KVH, T, hd):
    from nanonemo_b200.ops.attention import bwd_raw, fwd_raw
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(2)
    q = torch.randn(B, T, H, hd, device=DEV).bfloat16()
    k, v = torch.randn(B, T, KVH, hd, device=DEV).bfloat16(), torch.randn(B, T, KVH, hd, device=DEV).bfloat16()
    do = torch.randn(B, T, H, hd, device=DEV).bfloat16()

    def guarded4(heads):  # [B, T, heads, hd] view with sentinel rows before and after every batch entry's tokens
        big = torch.full((B, T + 4, heads, hd), SENTINEL, dtype=torch.bfloat16, device=DEV)
        view = big[:, 2:T + 2]
        view.fill_(float("nan"))
        return big, view

    def check4(big, view):
        edges = torch.cat((big[:, :2].flatten(), big[:, T + 2:].flatten()))
        assert torch.equal(edges, torch.full_like(edges, SENTINEL)) and not torch.isnan(view.float()).any()

    big_o, o = guarded4(H)
    lse = fwd_raw(q, k, v, o, 1.0 / math.sqrt(hd))
    check_status()
    check4(big_o, o)
    assert torch.isfinite(lse).all()
    (big_dq, dq), (big_dk, dk), (big_dv, dv) = guarded4(H), guarded4(KVH), guarded4(KVH)
    bwd_raw(q, k, v, o, lse, do, dq, dk, dv, 1.0 / math.sqrt(hd))
    check_status()
    for big, view in ((big_dq, dq), (big_dk, dk), (big_dv, dv)):
        check4(big, view)


def test_fixed_order_kernels_are_bitwise_reproducible():
    from nanonemo_b200 import ops
    from nanonemo_b200.ops.attention import bwd_raw, fwd_raw
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(3)
    a, b = torch.randn(4096, 768, device=DEV).bfloat16(), torch.randn(1280, 768, device=DEV).bfloat16()
    bt = torch.randn(768, 1280, device=DEV).bfloat16()
    for bn in (0, 256):
        assert torch.equal(gemm(a, b, bn=bn), gemm(a, b, bn=bn))
        assert torch.equal(gemm(a, bt, b_mn=True, bn=bn), gemm(a, bt, b_mn=True, bn=bn))
    B, T, H, KVH, hd = 2, 512, 6, 2, 64
    q = torch.randn(B, T, H, hd, device=DEV).bfloat16()
    k, v = torch.randn(B, T, KVH, hd, device=DEV).bfloat16(), torch.randn(B, T, KVH, hd, device=DEV).bfloat16()
    do = torch.randn(B, T, H, hd, device=DEV).bfloat16()
    runs = []
    for _ in range(2):
        o = torch.empty_like(q)
        lse = fwd_raw(q, k, v, o, 0.125)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        bwd_raw(q, k, v, o, lse, do, dq, dk, dv, 0.125)
        runs.append((o, lse, dk, dv))  # dQ is summed over key tiles by reduce-adds in arrival order: tolerance-tested elsewhere
    check_status()
    for x, y in zip(*runs):
        assert torch.equal(x, y)
    x = torch.randn(2048, 768, device=DEV)
    d = torch.randn(2048, 768, device=DEV).bfloat16()
    w = torch.rand(768, device=DEV) + 0.5
    n1, n2 = ops.add_rms_norm(x, d, w, 1e-5, impl="sm100"), ops.add_rms_norm(x, d, w, 1e-5, impl="sm100")
    assert all(torch.equal(p, q_) for p, q_ in zip(n1, n2))
    h = (torch.randn(1024, 256, device=DEV) * 0.5).bfloat16()
    wt = torch.randn(2048, 256, device=DEV) * 0.1
    t = torch.randint(0, 2048, (1024,), device=DEV)
    assert torch.equal(ops.linear_cross_entropy(h, wt, t), ops.linear_cross_entropy(h, wt, t))
