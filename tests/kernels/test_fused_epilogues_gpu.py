"""GEMM epilogue fusions (SwiGLU, RoPE, softmax statistics) and the inverse RoPE inside the attention backward, each
against the unfused composition of the same operators and against plain fp32 PyTorch math."""

import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(out, ref, tol=2e-2):
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * scale + 1e-3, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("M,F_,K", [(256, 128, 64), (512, 256, 768), (1000, 512, 264), (4096, 2048, 768), (384, 5632, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_swiglu_epilogue(M, F_, K, dtype):
    from nanonemo_b200.ops.gemm import check_status, gemm_swiglu

    torch.manual_seed(M + F_ + K)
    x = torch.randn(M, K, device=DEV).to(dtype)
    w = (torch.randn(2 * F_, K, device=DEV) / math.sqrt(K)).to(dtype)
    res = gemm_swiglu(x, w)
    check_status()
    assert res is not None
    gu, act = res
    _close(gu, x.float() @ w.float().t())
    g, u = gu.float().split(F_, dim=1)
    _close(act, F.silu(g) * u, tol=1e-2)  # from the ROUNDED projection, as the stand-alone kernel computes it


def test_gemm_swiglu_declines_shapes_it_does_not_serve():
    from nanonemo_b200.ops.gemm import gemm_swiglu

    x = torch.randn(128, 64, device=DEV).bfloat16()
    assert gemm_swiglu(x, torch.randn(256, 64, device=DEV).bfloat16()) is None          # fewer than 256 rows
    x = torch.randn(512, 64, device=DEV).bfloat16()
    assert gemm_swiglu(x, torch.randn(2 * 192, 64, device=DEV).bfloat16()) is None      # d_ff not a multiple of 128


@pytest.mark.parametrize("B,T,H,KVH,hd,K", [(2, 128, 4, 2, 64, 256), (3, 100, 12, 4, 64, 768), (2, 256, 16, 4, 128, 512),
                                             (1, 384, 2, 1, 128, 64), (4, 64, 5, 5, 64, 136)])
def test_gemm_rope_epilogue(B, T, H, KVH, hd, K):
    from nanonemo_b200 import ops
    from nanonemo_b200.models.layers import rope_cache
    from nanonemo_b200.ops.gemm import check_status, gemm, gemm_rope

    torch.manual_seed(B + T + H)
    N = (H + 2 * KVH) * hd
    x = torch.randn(B * T, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    cos, sin = rope_cache(hd, T, device=DEV)
    out = gemm_rope(x, w, cos.contiguous(), sin.contiguous(), T, (H + KVH) * hd, hd)
    check_status()
    assert out is not None
    plain = gemm(x, w)
    ref = ops.rope_qkv(plain.view(B, T, N), cos, sin, H, KVH, hd, impl="torch").view(B * T, N)
    _close(out, ref, tol=1e-2)
    assert torch.equal(out[:, (H + KVH) * hd:], plain[:, (H + KVH) * hd:])  # V passes through untouched
    unfused = ops.rope_qkv(plain.view(B, T, N), cos, sin, H, KVH, hd, impl="sm100").view(B * T, N)
    assert (out.float() - unfused.float()).abs().max().item() <= 2 ** -6 * unfused.float().abs().max().item()


@pytest.mark.parametrize("M,V,K", [(256, 512, 64), (512, 50304, 256), (1000, 25152, 128), (384, 1280, 768)])
def test_gemm_ce_stats_epilogue_and_one_sweep_ce(M, V, K):
    from nanonemo_b200.ops.gemm import check_status, gemm_ce_stats
    from nanonemo_b200.ops.linear_ce import ce_from_stats, ce_inplace

    torch.manual_seed(M + V)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(V, K, device=DEV) / math.sqrt(K) * 3).bfloat16()
    t = torch.randint(0, V, (M,), device=DEV)
    t[::7] = -100  # ignored rows
    logits = torch.empty(M, V, device=DEV, dtype=torch.bfloat16)
    stats = gemm_ce_stats(x, w, logits)
    check_status()
    assert stats is not None and stats.shape == (M, 2 * ((V + 255) // 256), 2)  # two parts per 256-column tile
    _close(logits, x.float() @ w.float().t())
    lf = logits.float()
    lse_tiles = stats[..., 0] + stats[..., 1].log()
    assert torch.allclose(torch.logsumexp(lse_tiles, dim=1), torch.logsumexp(lf, dim=1), atol=2e-3, rtol=0)
    # one sweep with the statistics == two sweeps without them
    two = logits.clone()
    loss_two, loss_one = torch.empty(M, device=DEV), torch.empty(M, device=DEV)
    ce_inplace(two, t, loss_two, 0.5)
    ce_from_stats(logits, t, stats, loss_one, 0.5)
    assert torch.allclose(loss_one, loss_two, atol=2e-3, rtol=0)
    assert (logits.float() - two.float()).abs().max().item() <= 1e-3
    valid = t >= 0
    ref_loss = F.cross_entropy(lf[valid], t[valid], reduction="none")
    assert torch.allclose(loss_one[valid], ref_loss, atol=5e-3, rtol=0)
    assert loss_one[~valid].abs().max().item() == 0
    ref_grad = (torch.softmax(lf, dim=1) - F.one_hot(t.clamp(min=0), V)) * 0.5 * valid[:, None]
    assert (logits.float() - ref_grad).abs().max().item() <= 4e-3


def test_linear_ce_same_result_with_and_without_the_stats_epilogue():
    from nanonemo_b200 import ops
    from nanonemo_b200.ops import linear_ce

    torch.manual_seed(0)
    x0 = torch.randn(1024, 256, device=DEV, dtype=torch.bfloat16)
    w0 = torch.randn(50304, 256, device=DEV) * 0.02
    t = torch.randint(0, 50257, (1024,), device=DEV)
    res = {}
    for fuse in (True, False):
        linear_ce.FUSE_STATS = fuse
        try:
            x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
            loss = ops.linear_cross_entropy(x, w, t)
            (loss * 0.5).backward()
            res[fuse] = (loss.item(), x.grad.float(), w.grad.float())
        finally:
            linear_ce.FUSE_STATS = True
    assert res[True][0] == pytest.approx(res[False][0], abs=1e-3)
    for a, b in zip(res[True][1:], res[False][1:]):
        assert (a - b).norm().item() <= 1e-2 * b.norm().item()


@pytest.mark.parametrize("B,T,H,KVH", [(2, 256, 4, 2), (1, 200, 12, 4)])
def test_flash_backward_with_inverse_rope_inside(B, T, H, KVH):
    from nanonemo_b200.models.layers import rope_cache
    from nanonemo_b200.ops import attention, rope
    from nanonemo_b200.ops.gemm import check_status

    hd = 64
    torch.manual_seed(T)
    C = (H + 2 * KVH) * hd
    qkv = torch.randn(B, T, C, device=DEV).bfloat16()
    do = torch.randn(B, T, H, hd, device=DEV).bfloat16()
    cos, sin = (t.contiguous() for t in rope_cache(hd, T, device=DEV))

    def split(t):
        return (t[..., : H * hd].view(B, T, H, hd), t[..., H * hd:(H + KVH) * hd].view(B, T, KVH, hd), t[..., (H + KVH) * hd:].view(B, T, KVH, hd))

    q, k, v = split(qkv)
    o = torch.empty(B, T, H, hd, device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    lse = attention.fwd_raw(q, k, v, o, scale)
    g_plain, g_fused = torch.empty_like(qkv), torch.empty_like(qkv)
    attention.bwd_raw(q, k, v, o, lse, do, *split(g_plain), scale)
    attention.bwd_raw(q, k, v, o, lse, do, *split(g_fused), scale, rope_cos=cos, rope_sin=sin)
    check_status()
    ref = torch.empty_like(g_plain)
    rope.rope_packed_raw(g_plain.view(B * T, C), ref.view(B * T, C), cos, sin, T, H + KVH, hd, KVH * hd, -1.0)
    _close(g_fused, ref, tol=1e-2)
    assert torch.equal(g_fused[..., (H + KVH) * hd:], g_plain[..., (H + KVH) * hd:])  # dV is not rotated


SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, d_ff=512, vocab_size=50304, max_seq_len=256)


@pytest.mark.parametrize("shape", ["hd64", "hd128"])
def test_model_same_loss_and_gradients_with_and_without_fused_epilogues(shape):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.models.model import NanoNemo
    from nanonemo_b200.ops.gemm import check_status

    extra = {} if shape == "hd64" else dict(n_heads=2, n_kv_heads=1, head_dim_override=128)
    idx = torch.randint(0, 50257, (4, 257), device=DEV)
    out = {}
    for fuse in (True, False):
        torch.manual_seed(0)
        model = NanoNemo(ModelConfig.sm100(**{**SMALL, **extra}, fuse_epilogues=fuse)).to(DEV)
        assert model.blocks[0].attn.fused == fuse and model.blocks[0].mlp.fused == fuse
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = model(idx[:, :-1], idx[:, 1:])
        loss.backward()
        out[fuse] = (loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()})
    check_status()
    assert out[True][0] == pytest.approx(out[False][0], abs=2e-3)
    for n, g in out[True][1].items():
        ref = out[False][1][n]
        assert (g - ref).norm().item() <= 2e-2 * ref.norm().item() + 1e-8, n


@pytest.mark.parametrize("M,F_,K", [(256, 128, 64), (512, 256, 768), (1000, 512, 264), (4096, 2048, 768), (384, 5632, 128), (640, 192, 96)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_swiglu_backward_epilogue(M, F_, K, dtype):
    """d(gate) | d(up) written by the epilogue of dy @ W_down against fp32 math on the same (rounded) saved projection."""
    from nanonemo_b200.ops.gemm import check_status, gemm_swiglu_bwd

    torch.manual_seed(M + F_ + K)
    dy = torch.randn(M, K, device=DEV).to(dtype)
    w_down = (torch.randn(K, F_, device=DEV) / math.sqrt(K)).to(dtype)  # [d_model, d_ff] as the layer stores it
    gu = torch.randn(M, 2 * F_, device=DEV).to(dtype)
    dgu = gemm_swiglu_bwd(dy, w_down, gu)
    check_status()
    assert dgu is not None and dgu.shape == (M, 2 * F_)
    dact = dy.float() @ w_down.float()
    g, u = gu.float().split(F_, dim=1)
    s = torch.sigmoid(g)
    _close(dgu[:, :F_], dact * u * s * (1 + g * (1 - s)))
    _close(dgu[:, F_:], dact * g * s)
    # twice in a row: the staging pairs and their barriers carry over from tile to tile and from launch to launch
    assert torch.equal(dgu, gemm_swiglu_bwd(dy, w_down, gu))


def test_mlp_node_matches_unfused_composition():
    """The one-node feed-forward (SwiGLU backward inside the down projection's dgrad) against linear -> swiglu -> linear built
    from the separate operators, and against fp32 PyTorch: output, input gradient and both weight gradients."""
    from nanonemo_b200.ops import fused_block
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(11)
    M, d, F_ = 1024, 256, 512
    x = torch.randn(4, M // 4, d, device=DEV).bfloat16().requires_grad_()
    w_gu = (torch.randn(2 * F_, d, device=DEV) / math.sqrt(d)).requires_grad_()
    w_down = (torch.randn(d, F_, device=DEV) / math.sqrt(F_)).requires_grad_()
    g_out = torch.randn(4, M // 4, d, device=DEV).bfloat16()
    results = {}
    for fused in (True, False):
        fused_block.FUSE_SWIGLU_BWD = fused
        for t in (x, w_gu, w_down):
            t.grad = None
        y = fused_block.mlp_swiglu(x, w_gu, w_down)
        y.backward(g_out)
        check_status()
        results[fused] = (y.detach().clone(), x.grad.clone(), w_gu.grad.clone(), w_down.grad.clone())
    fused_block.FUSE_SWIGLU_BWD = True
    xr, wgr, wdr = (t.detach().float().requires_grad_() for t in (x, w_gu.bfloat16(), w_down.bfloat16()))
    gate, up = (xr @ wgr.t()).split(F_, dim=-1)
    ref = (F.silu(gate) * up) @ wdr.t()
    ref.backward(g_out.float())
    for got_f, got_u, want in zip(results[True], results[False], (ref, xr.grad, wgr.grad, wdr.grad)):
        _close(got_f, want, tol=3e-2)
        _close(got_f, got_u, tol=2e-2)
