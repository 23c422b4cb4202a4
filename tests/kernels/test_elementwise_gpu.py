"""GPU parity of the bandwidth-bound sm100 kernels against plain PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ref_add_rms(x, delta, w, eps):
    h = x if delta is None else (x.float() + delta.float()).to(x.dtype)
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y, h


@pytest.mark.parametrize("M,N", [(1, 8), (7, 768), (64, 768), (33, 1000), (16, 2048), (5, 72)])
@pytest.mark.parametrize("xd,cd", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                   (torch.bfloat16, torch.bfloat16), (torch.float32, torch.float16)])
@pytest.mark.parametrize("has_delta", [True, False])
def test_add_rms_norm_fwd_bwd(M, N, xd, cd, has_delta):
    from nanonemo_b200.ops import rmsnorm

    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, N, device=DEV).to(xd).requires_grad_()
    delta = torch.randn(M, N, device=DEV).to(cd).requires_grad_() if has_delta else None
    w = (1 + 0.1 * torch.randn(N, device=DEV)).requires_grad_()
    y, h, rstd = rmsnorm._AddRMSNorm.apply(x, delta, w, 1e-5)
    assert y.dtype == (cd if has_delta else xd) and h.dtype == xd
    xr = x.detach().clone().requires_grad_()
    dr = delta.detach().clone().requires_grad_() if has_delta else None
    wr = w.detach().clone().requires_grad_()
    yr, hr = _ref_add_rms(xr, dr, wr, 1e-5)
    tol = 1e-5 if y.dtype == torch.float32 else 2e-2
    torch.testing.assert_close(y.float(), yr.float(), rtol=tol, atol=tol)
    torch.testing.assert_close(h.float(), hr.float(), rtol=1e-6 if xd == torch.float32 else 1e-2, atol=1e-6 if xd == torch.float32 else 1e-2)
    gy = torch.randn_like(yr).to(y.dtype)
    gh = torch.randn_like(hr).to(h.dtype)
    torch.autograd.backward([y, h], [gy, gh])
    torch.autograd.backward([yr, hr], [gy.to(yr.dtype), gh.to(hr.dtype)])
    gtol = 2e-4 if y.dtype == torch.float32 and xd == torch.float32 else 4e-2
    torch.testing.assert_close(x.grad.float(), xr.grad.float(), rtol=gtol, atol=gtol)
    if has_delta:
        torch.testing.assert_close(delta.grad.float(), dr.grad.float(), rtol=gtol, atol=gtol)
    torch.testing.assert_close(w.grad, wr.grad, rtol=gtol, atol=gtol * max(1.0, M ** 0.5))


@pytest.mark.parametrize("B,T,H,KVH,hd", [(2, 16, 4, 2, 32), (1, 33, 12, 4, 64), (3, 8, 16, 4, 128), (2, 5, 2, 2, 16)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_rope_qkv(B, T, H, KVH, hd, dtype):
    from nanonemo_b200 import ops
    from nanonemo_b200.models.layers import rope_cache

    torch.manual_seed(0)
    cos, sin = rope_cache(hd, 64, device=DEV)
    C = (H + 2 * KVH) * hd
    qkv = torch.randn(B, T, C, device=DEV).to(dtype).requires_grad_()
    ref_in = qkv.detach().float().requires_grad_()
    out = ops.rope_qkv(qkv, cos, sin, H, KVH, hd, impl="sm100")
    ref = ops.rope_qkv(ref_in, cos, sin, H, KVH, hd, impl="torch")
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(out.float(), ref, rtol=tol, atol=tol)
    g = torch.randn_like(ref)
    out.backward(g.to(dtype))
    ref.backward(g)
    torch.testing.assert_close(qkv.grad.float(), ref_in.grad, rtol=tol, atol=tol)
    # inverse round trip: rotating by -theta restores the input
    from nanonemo_b200.ops.rope import rope_packed_raw

    x2 = qkv.detach().reshape(B * T, C)
    y2, z2 = torch.empty_like(x2), torch.empty_like(x2)
    rope_packed_raw(x2, y2, cos[:T].contiguous(), sin[:T].contiguous(), T, H + KVH, hd, KVH * hd, 1.0)
    rope_packed_raw(y2, z2, cos[:T].contiguous(), sin[:T].contiguous(), T, H + KVH, hd, KVH * hd, -1.0)
    torch.testing.assert_close(z2.float(), x2.float(), rtol=tol, atol=tol)


def test_rope_strided_front_end():
    from nanonemo_b200 import ops
    from nanonemo_b200.models.layers import rope_cache

    cos, sin = rope_cache(64, 32, device=DEV)
    big = torch.randn(2, 12, 6, 128, device=DEV, dtype=torch.bfloat16)
    q, k = big[:, :, :4, :64], big[:, :, 4:, 64:]  # strided views
    q1, k1 = ops.apply_rope_qk(q, k, cos, sin, impl="sm100")
    q0, k0 = ops.apply_rope_qk(q.float(), k.float(), cos, sin, impl="torch")
    torch.testing.assert_close(q1.float(), q0, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(k1.float(), k0, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,F", [(1, 8), (17, 2048), (128, 384), (3, 5632)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_swiglu(M, F, dtype):
    from nanonemo_b200 import ops

    torch.manual_seed(1)
    gu = torch.randn(M, 2 * F, device=DEV).to(dtype).requires_grad_()
    ref_in = gu.detach().float().requires_grad_()
    out = ops.swiglu_packed(gu, impl="sm100")
    ref = ops.swiglu_packed(ref_in, impl="torch")
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(out.float(), ref, rtol=tol, atol=tol)
    g = torch.randn_like(ref)
    out.backward(g.to(dtype))
    ref.backward(g)
    torch.testing.assert_close(gu.grad.float(), ref_in.grad, rtol=tol, atol=tol)
    a, b = torch.randn(M, F, device=DEV).to(dtype), torch.randn(M, F, device=DEV).to(dtype)
    torch.testing.assert_close(ops.swiglu(a, b, impl="sm100").float(), ops.swiglu(a.float(), b.float()), rtol=tol, atol=tol)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_embedding(out_dtype):
    from nanonemo_b200.ops.embed import embedding

    torch.manual_seed(2)
    W = torch.randn(1000, 64, device=DEV, requires_grad=True)
    idx = torch.randint(0, 1000, (4, 37), device=DEV)
    idx[0, :5] = 7  # repeated rows must add up
    out = embedding(idx, W, out_dtype)
    ref = torch.nn.functional.embedding(idx, W.detach())
    torch.testing.assert_close(out.float(), ref, rtol=1e-2 if out_dtype != torch.float32 else 0, atol=1e-2 if out_dtype != torch.float32 else 0)
    g = torch.randn_like(ref)
    out.backward(g.to(out_dtype))
    Wr = W.detach().clone().requires_grad_()
    torch.nn.functional.embedding(idx, Wr).backward(g.to(out_dtype).float())
    torch.testing.assert_close(W.grad, Wr.grad, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n", [1, 255, 256, 1000, 1 << 20])
def test_warmup_add(n):
    from nanonemo_b200.ops.warmup import warmup_add

    a, b = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
    assert torch.equal(warmup_add(a, b), a + b)
    with pytest.raises(TypeError):
        warmup_add(a.half(), b.half())


@pytest.mark.parametrize("n", [256, 4096, 3 * 1024 * 1024 + 256])
def test_sumsq_and_adamw_match_torch(n):
    from nanonemo_b200.ops.adamw import adamw_flat, sumsq

    torch.manual_seed(3)
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 3
    ss = sumsq(g)
    torch.testing.assert_close(ss, g.double().pow(2).sum().float(), rtol=1e-5, atol=0)
    assert torch.equal(sumsq(g), ss)  # deterministic
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    flags = torch.ones(n // 256, dtype=torch.uint8, device=DEV)
    shadow = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    for step in range(1, 4):
        gstep = g * step
        ref_p.grad = gstep.clone()
        norm = torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        gbuf = gstep.clone()
        adamw_flat(p, gbuf, m, v, shadow, flags, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                   grad_norm_sq=sumsq(gbuf), max_norm=1.0, zero_grad=True)
        assert gbuf.abs().max() == 0
        torch.testing.assert_close(p, ref_p.data, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(shadow.float(), ref_p.data, rtol=1e-2, atol=1e-2)
