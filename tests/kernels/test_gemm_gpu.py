"""tcgen05 GEMM against fp32 matmul: the three operand layouts, tails, split-K, accumulate."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= 2e-2 * scale + 1e-3, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (256, 512, 768), (384, 1280, 768), (130, 264, 72),
                                   (1000, 768, 2048), (64, 64, 64), (4096, 768, 768), (2560, 20096, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fprop_layout(M, N, K, dtype):
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(dtype)
    b = torch.randn(N, K, device=DEV).to(dtype)
    out = gemm(a, b)
    check_status()
    _check(out, _ref(a, b, False, False), K)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 768, 1280), (384, 2048, 768), (200, 136, 264)])
def test_dgrad_layout(M, N, K):
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV).bfloat16()
    bt = torch.randn(K, N, device=DEV).bfloat16()  # B stored transposed
    out = gemm(a, bt, b_mn=True)
    check_status()
    _check(out, _ref(a, bt, False, True), K)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1280, 768, 4096), (768, 2048, 1024), (136, 72, 520)])
@pytest.mark.parametrize("k_splits", [0, 1, 3])
def test_wgrad_layout_fp32_out(M, N, K, k_splits):
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(2)
    at = torch.randn(K, M, device=DEV).bfloat16()
    bt = torch.randn(K, N, device=DEV).bfloat16()
    ref = _ref(at, bt, True, True)
    out = gemm(at, bt, a_mn=True, b_mn=True, out_dtype=torch.float32, k_splits=k_splits)
    check_status()
    _check(out, ref, K)
    acc = torch.ones(M, N, device=DEV)
    gemm(at, bt, a_mn=True, b_mn=True, out=acc, accumulate=True, k_splits=k_splits)
    check_status()
    _check(acc - 1, ref, K)


@pytest.mark.parametrize("layout", ["fprop", "dgrad", "wgrad"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 768), (1024, 2304, 768), (384, 1280, 1024), (2048, 256, 2048),
                                   (304, 520, 136), (4096, 4352, 128), (21504, 256, 64), (32768, 768, 128), (21760, 520, 72)])
def test_cta_pair_kernel(layout, M, N, K):
    """bn=512 selects the two-SM kernel (256 x 256 tiles, tcgen05.mma.cta_group::2); ragged edges and an odd number of
    128-row blocks (the second CTA's last block lies outside the matrix) included; the three tall shapes leave a tail wave of
    at most half the CTA pairs, which the kernel works on as 128-wide half tiles."""
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(M + N + K)
    if layout == "fprop":
        a, b = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(N, K, device=DEV).bfloat16()
        out, ref = gemm(a, b, bn=512), _ref(a, b, False, False)
    elif layout == "dgrad":
        a, b = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(K, N, device=DEV).bfloat16()
        out, ref = gemm(a, b, b_mn=True, bn=512), _ref(a, b, False, True)
    else:
        a, b = torch.randn(K, M, device=DEV).bfloat16(), torch.randn(K, N, device=DEV).bfloat16()
        ref = _ref(a, b, True, True)
        out = gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32, bn=512)
        acc = torch.ones(M, N, device=DEV)
        gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, k_splits=2 if K >= 128 else 1, bn=512)
        check_status()
        _check(acc - 1, ref, K)
    check_status()
    _check(out, ref, K)


def test_strided_views_and_bn128():
    from nanonemo_b200.ops.gemm import check_status, gemm

    big = torch.randn(300, 2048, device=DEV).bfloat16()
    a = big[:, 512:1280]  # row stride 2048, 16-byte aligned offset
    b = torch.randn(768, 768, device=DEV).bfloat16()
    for bn in (128, 192, 256):
        out = gemm(a, b, bn=bn)
        check_status()
        _check(out, _ref(a, b, False, False), 768)


def test_linear_autograd_matches_torch():
    from nanonemo_b200.ops.gemm import check_status, linear_sm100

    torch.manual_seed(3)
    x = torch.randn(4, 96, 768, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(1280, 768, device=DEV) * 0.02).requires_grad_()
    y = linear_sm100(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    check_status()
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    _check(y, yr, 768)
    _check(x.grad, xr.grad, 1280)
    _check(w.grad, wr.grad, 384)
