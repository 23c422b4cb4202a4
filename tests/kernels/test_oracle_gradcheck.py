"""fp64 ``gradcheck`` of the PyTorch oracles that every kernel is tested against (CPU). The kernels themselves have no fp64
path (the reference's Triton kernels do, tests/kernels/test_rope.py:65-67, test_swiglu.py:40-42), so the chain is: the
oracle's analytic gradients match finite differences in fp64 here, and the kernels' gradients match the oracle's on the GPU
(tests/kernels/test_elementwise_gpu.py, test_flash_attn_gpu.py, test_linear_ce_model_gpu.py)."""

import torch
from torch.autograd import gradcheck

from nanonemo_b200 import ops
from nanonemo_b200.models.layers import rope_cache


def _d(*shape):
    return torch.randn(*shape, dtype=torch.float64, requires_grad=True)


def test_add_rms_norm_oracle():
    torch.manual_seed(0)
    x, d, w = _d(3, 5, 16), _d(3, 5, 16), _d(16)
    assert gradcheck(lambda x, d, w: ops.add_rms_norm_torch(x, d, w, 1e-5), (x, d, w), eps=1e-6, atol=1e-5)
    assert gradcheck(lambda x, w: ops.add_rms_norm_torch(x, None, w, 1e-5)[0], (x, w), eps=1e-6, atol=1e-5)


def test_rope_oracle_and_its_inverse():
    torch.manual_seed(1)
    cos, sin = (t.double() for t in rope_cache(8, 6))
    x = _d(2, 6, 3, 8)
    assert gradcheck(lambda x: ops.rope_torch(x, cos, sin, seq_dim=1), (x,), eps=1e-6, atol=1e-6)
    y = ops.rope_torch(x, cos, sin, seq_dim=1)
    assert torch.allclose(ops.rope_torch(y, cos, -sin, seq_dim=1), x, atol=1e-12)  # negated sine = inverse = backward


def test_swiglu_oracle():
    torch.manual_seed(2)
    g, u = _d(4, 12), _d(4, 12)
    assert gradcheck(ops.swiglu_torch, (g, u), eps=1e-6, atol=1e-6)
    # the recompute-sigma formulas the kernels use (nanonemo/kernels/triton/swiglu.py:45-66)
    dy = torch.randn(4, 12, dtype=torch.float64)
    dg, du = torch.autograd.grad(ops.swiglu_torch(g, u), (g, u), dy)
    s = torch.sigmoid(g)
    assert torch.allclose(dg, dy * u * s * (1 + g * (1 - s)), atol=1e-12) and torch.allclose(du, dy * g * s, atol=1e-12)


def test_attention_and_linear_ce_oracles():
    torch.manual_seed(3)
    q, k, v = _d(1, 4, 5, 4), _d(1, 2, 5, 4), _d(1, 2, 5, 4)
    assert gradcheck(ops.attention_torch, (q, k, v), eps=1e-6, atol=1e-5)
    x, w = _d(6, 8), _d(10, 8)
    t = torch.tensor([1, 0, 9, 3, 3, 7])
    assert gradcheck(lambda x, w: ops.linear_cross_entropy_torch(x, w, t), (x, w), eps=1e-6, atol=1e-5)
