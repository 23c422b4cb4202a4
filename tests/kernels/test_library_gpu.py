"""torch.library surface: opcheck (schema, fake tensor, autograd registration) and fullgraph compile."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_opcheck_every_registered_operator():
    from nanonemo_b200.models.layers import rope_cache
    from nanonemo_b200.ops import library as L

    torch.manual_seed(0)
    bf = torch.bfloat16
    x = torch.randn(2, 16, 128, device=DEV, requires_grad=True)
    d = torch.randn(2, 16, 128, device=DEV, dtype=bf, requires_grad=True)
    w = torch.ones(128, device=DEV, requires_grad=True)
    torch.library.opcheck(L.add_rms_norm, (x, d, w, 1e-5))
    gu = torch.randn(4, 32, 256, device=DEV, dtype=bf, requires_grad=True)
    torch.library.opcheck(L.swiglu, (gu,))
    cos, sin = rope_cache(64, 128, device=DEV)
    qkv = torch.randn(2, 128, (4 + 2 * 2) * 64, device=DEV, dtype=bf, requires_grad=True)
    torch.library.opcheck(L.rope_qkv, (qkv, cos, sin, 4, 2, 64))
    torch.library.opcheck(L.flash_attn_packed, (qkv, 4, 2, 64))
    a = torch.randn(256, 128, device=DEV, dtype=bf, requires_grad=True)
    b = torch.randn(384, 128, device=DEV, dtype=bf, requires_grad=True)
    torch.library.opcheck(L.matmul_nt, (a, b))


def test_registered_ops_match_the_direct_functions():
    from nanonemo_b200 import ops
    from nanonemo_b200.ops import library as L

    torch.manual_seed(1)
    qkv = torch.randn(2, 256, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o1, _ = L.flash_attn_packed(qkv, 4, 2, 64)
    o2 = ops.attention_packed(qkv, 4, 2, 64, impl="sm100")
    assert torch.equal(o1, o2)
    g = torch.randn_like(o1)
    (g1,) = torch.autograd.grad(o1, qkv, g)
    (g2,) = torch.autograd.grad(o2, qkv, g)
    torch.testing.assert_close(g1.float(), g2.float(), rtol=2e-2, atol=2e-2)  # dQ partials are reduce-added in arrival order


def test_fullgraph_compile_has_no_graph_break():
    from nanonemo_b200.ops import library as L

    def f(gu, qkv):
        return L.swiglu(gu).sum() + L.flash_attn_packed(qkv, 4, 2, 64)[0].float().sum()

    gu = torch.randn(8, 64, 256, device=DEV, dtype=torch.bfloat16)
    qkv = torch.randn(2, 128, 512, device=DEV, dtype=torch.bfloat16)
    try:
        compiled = torch.compile(f, fullgraph=True, backend="aot_eager")
        torch.testing.assert_close(compiled(gu, qkv), f(gu, qkv), rtol=1e-3, atol=1e-3)
    except RuntimeError as e:  # a compile toolchain problem on the box is not an operator bug
        if "fullgraph" in str(e) or "graph break" in str(e).lower():
            raise
        pytest.skip(f"torch.compile unavailable: {e}")
