"""FlashAttention (tcgen05) against PyTorch attention in fp32: MHA / GQA, odd T, hd 64 / 128."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(q, k, v):
    group = q.shape[1] // k.shape[1]
    qf, kf, vf = q.float(), k.float().repeat_interleave(group, 1), v.float().repeat_interleave(group, 1)
    T = q.shape[2]
    s = qf @ kf.transpose(-1, -2) / q.shape[-1] ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=q.device), 1), float("-inf"))
    return torch.softmax(s, -1) @ vf


@pytest.mark.parametrize("B,H,KVH,T,hd", [(1, 1, 1, 128, 64), (2, 4, 2, 256, 64), (1, 12, 4, 1024, 64), (2, 3, 1, 200, 64),
                                          (1, 2, 2, 37, 64), (1, 4, 1, 384, 128), (2, 2, 2, 100, 128), (1, 2, 1, 640, 64)])
def test_forward_matches_reference(B, H, KVH, T, hd):
    from nanonemo_b200 import ops
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(T + hd)
    q = torch.randn(B, H, T, hd, device=DEV).bfloat16()
    k = torch.randn(B, KVH, T, hd, device=DEV).bfloat16()
    v = torch.randn(B, KVH, T, hd, device=DEV).bfloat16()
    out = ops.flash_attn(q, k, v)
    check_status()
    assert out.shape == (B, H, T, hd)
    torch.testing.assert_close(out.float(), _ref(q, k, v), rtol=2e-2, atol=2e-2)


def test_future_keys_do_not_leak():
    from nanonemo_b200 import ops

    torch.manual_seed(0)
    q = torch.randn(1, 2, 256, 64, device=DEV).bfloat16()
    k = torch.randn(1, 2, 256, 64, device=DEV).bfloat16()
    v = torch.randn(1, 2, 256, 64, device=DEV).bfloat16()
    a = ops.flash_attn(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 150:] = 100.0
    v2[:, :, 150:] = -100.0
    b = ops.flash_attn(q, k2, v2)
    assert torch.equal(a[:, :, :150], b[:, :, :150])  # bitwise: positions before 150 never read later keys


def test_packed_forward_and_backward():
    from nanonemo_b200 import ops
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(1)
    B, T, H, KVH, hd = 2, 384, 6, 2, 64
    qkv = torch.randn(B, T, (H + 2 * KVH) * hd, device=DEV).bfloat16().requires_grad_()
    out = ops.attention_packed(qkv, H, KVH, hd, impl="sm100")
    ref_in = qkv.detach().float().requires_grad_()
    ref = ops.attention_packed(ref_in, H, KVH, hd, impl="torch")
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(ref)
    out.backward(g.bfloat16())
    ref.backward(g)
    check_status()
    torch.testing.assert_close(qkv.grad.float(), ref_in.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("B,H,KVH,T,hd", [(1, 2, 1, 256, 64), (2, 6, 2, 512, 64), (1, 3, 3, 200, 64), (1, 4, 2, 1024, 64),
                                          (1, 1, 1, 128, 128), (1, 2, 1, 256, 128), (2, 4, 2, 512, 128), (1, 3, 3, 200, 128),
                                          (1, 4, 1, 1024, 128), (1, 2, 2, 37, 128)])
def test_backward_matches_reference(B, H, KVH, T, hd):
    from nanonemo_b200 import ops
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(2)
    q = torch.randn(B, H, T, hd, device=DEV).bfloat16().requires_grad_()
    k = torch.randn(B, KVH, T, hd, device=DEV).bfloat16().requires_grad_()
    v = torch.randn(B, KVH, T, hd, device=DEV).bfloat16().requires_grad_()
    out = ops.flash_attn(q, k, v)
    g = torch.randn(B, H, T, hd, device=DEV)
    out.backward(g.bfloat16())
    check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    _ref(qr, kr, vr).backward(g.bfloat16().float())
    for got, want, name in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk"), (v.grad, vr.grad, "dv")):
        err = (got.float() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 2e-2, f"{name}: max err {err}"


@pytest.mark.parametrize("B,H,KVH,T,hd", [(2, 4, 2, 256, 64), (1, 3, 1, 200, 64), (1, 4, 1, 384, 128), (1, 2, 2, 37, 128)])
def test_fp16_operands_run_natively(B, H, KVH, T, hd):
    """fp16 q / k / v go to the tensor cores as fp16 (no bf16 detour): forward and the three gradients against the fp32
    reference, with the tighter tolerance the 10-bit mantissa allows."""
    from nanonemo_b200 import ops
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(3)
    q = torch.randn(B, H, T, hd, device=DEV).half().requires_grad_()
    k = torch.randn(B, KVH, T, hd, device=DEV).half().requires_grad_()
    v = torch.randn(B, KVH, T, hd, device=DEV).half().requires_grad_()
    out = ops.flash_attn(q, k, v)
    assert out.dtype == torch.float16
    g = torch.randn(B, H, T, hd, device=DEV).half()
    out.backward(g)
    check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref(qr, kr, vr)
    ref.backward(g.float())
    torch.testing.assert_close(out.float(), ref, rtol=4e-3, atol=4e-3)
    for got, want, name in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk"), (v.grad, vr.grad, "dv")):
        assert got.dtype == torch.float16
        err = (got.float() - want).abs().max().item()
        assert err <= 6e-3 * want.abs().max().item() + 4e-3, f"{name}: max err {err}"


def test_mixed_operand_dtypes_are_refused():
    from nanonemo_b200.ops import attention

    q = torch.randn(1, 128, 1, 64, device=DEV).half()
    k = torch.randn(1, 128, 1, 64, device=DEV).bfloat16()
    with pytest.raises(TypeError):
        attention.fwd_raw(q, k, k, torch.empty_like(q), 0.125)
