"""torch.library surface: opcheck (schema, fake tensor, autograd registration) of EVERY registered operator, fullgraph
compile of the whole model on them, and that the model's sm100 path really is these operators."""

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
    g, u = (torch.randn(4, 32, 128, device=DEV, dtype=bf, requires_grad=True) for _ in range(2))
    torch.library.opcheck(L.swiglu_gu, (g, u))
    cos, sin = (t.contiguous() for t in rope_cache(64, 128, device=DEV))
    qkv = torch.randn(2, 128, (4 + 2 * 2) * 64, device=DEV, dtype=bf, requires_grad=True)
    torch.library.opcheck(L.rope_qkv, (qkv, cos, sin, 4, 2, 64))
    rows = torch.randn(256, 6 * 64, device=DEV, dtype=bf, requires_grad=True)
    torch.library.opcheck(L.rope_rows, (rows, cos, sin, 128, 4, 64, 1.0))
    torch.library.opcheck(L.flash_attn_packed, (qkv, 4, 2, 64))
    q = torch.randn(2, 128, 4, 64, device=DEV, dtype=bf).transpose(1, 2).requires_grad_()
    k, v = (torch.randn(2, 128, 2, 64, device=DEV, dtype=bf).transpose(1, 2).requires_grad_() for _ in range(2))
    torch.library.opcheck(L.flash_attn, (q, k, v), test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    a = torch.randn(256, 128, device=DEV, dtype=bf, requires_grad=True)
    b = torch.randn(384, 128, device=DEV, dtype=bf, requires_grad=True)
    torch.library.opcheck(L.matmul_nt, (a, b))
    w32 = (torch.randn(384, 128, device=DEV) * 0.05).requires_grad_()
    torch.library.opcheck(L.linear_w, (a, w32))
    wq = (torch.randn(8 * 64, 128, device=DEV) * 0.05).requires_grad_()
    torch.library.opcheck(L.gemm_rope, (a, wq, cos, sin, 128, 6 * 64, 64))
    wg = (torch.randn(2 * 128, 128, device=DEV) * 0.05).requires_grad_()
    torch.library.opcheck(L.gemm_swiglu, (a, wg))
    idx = torch.randint(0, 512, (4, 33), device=DEV)
    table = (torch.randn(512, 64, device=DEV) * 0.02).requires_grad_()
    torch.library.opcheck(L.embedding, (idx, table, True))
    head = (torch.randn(512, 128, device=DEV) * 0.02).requires_grad_()
    tg = torch.randint(0, 512, (256,), device=DEV)
    torch.library.opcheck(L.linear_ce, (a, head, tg, 128))
    n = 1024
    p, gr, m, vv = (torch.randn(n, device=DEV) for _ in range(4))
    vv.abs_()
    torch.library.opcheck(L.adamw_step, (p, gr, m, vv, torch.zeros(n, device=DEV, dtype=bf), torch.ones(n // 256, device=DEV, dtype=torch.uint8),
                                         torch.tensor(4.0, device=DEV), 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, 1.0, True))


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


def test_adamw_operator_matches_torch_adamw():
    from nanonemo_b200.ops import library as L

    torch.manual_seed(2)
    n = 4096
    p0, g0 = torch.randn(n, device=DEV), torch.randn(n, device=DEV) * 0.1
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    p, m, v = p0.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    shadow = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    flags = torch.ones(n // 256, device=DEV, dtype=torch.uint8)
    for step in range(1, 4):
        ref.grad = g0.clone()
        opt.step()
        g = g0.clone()
        L.adamw_step(p, g, m, v, shadow, flags, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.0, True)
        assert g.abs().max().item() == 0
    torch.testing.assert_close(p, ref.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(shadow.float(), p, rtol=1e-2, atol=1e-2)


SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, d_ff=512, vocab_size=50304, max_seq_len=256)


def test_whole_model_compiles_fullgraph_on_the_registered_operators():
    """A model outside a flat parameter store runs entirely on the registered operators: it traces with fullgraph=True (no
    graph break anywhere) and the traced module gives the eager loss and gradients."""
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.models.model import NanoNemo
    from nanonemo_b200.ops import direct

    direct.enable(False)  # (an earlier test of this process may have built a trainer engine, which switches the direct functions on)
    torch.manual_seed(0)
    model = NanoNemo(ModelConfig.sm100(**SMALL)).to(DEV)
    idx = torch.randint(0, 50257, (4, 257), device=DEV)

    def run(m):
        m.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = m(idx[:, :-1], idx[:, 1:])
        loss.backward()
        return loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()}

    eager_loss, eager_grads = run(model)
    try:
        compiled = torch.compile(model, fullgraph=True, backend="aot_eager")
        loss, grads = run(compiled)
    except RuntimeError as e:  # a compile toolchain problem on the box is not an operator bug
        if "fullgraph" in str(e) or "graph break" in str(e).lower():
            raise
        pytest.skip(f"torch.compile unavailable: {e}")
    assert loss == pytest.approx(eager_loss, abs=2e-3)
    for n, g in grads.items():
        assert (g - eager_grads[n]).norm().item() <= 2e-2 * eager_grads[n].norm().item() + 1e-8, n
