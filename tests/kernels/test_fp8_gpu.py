"""MXFP8 quantiser kernels and the fp8 linear: block-scale rules, round trip, and loss tracking vs bf16."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_quantise_matches_reference_rules():
    from nanonemo_b200 import fp8

    torch.manual_seed(0)
    x = (torch.randn(64, 256, device="cuda") * torch.logspace(-3, 2, 256, device="cuda")).bfloat16()
    q, s = fp8.quantize(x)
    assert q.shape == (64, 256) and s.shape == (64, 8)
    blocks = x.float().view(64, 8, 32)
    amax = blocks.abs().amax(-1)
    expect = (torch.floor(torch.log2(amax)) - 8 + 127).clamp(0, 254)
    assert torch.equal(s.float(), expect)
    deq = fp8.dequantize(q, s)
    torch.testing.assert_close(deq, fp8.fake_quant(x).float(), rtol=0, atol=0)
    rel = (deq - x.float()).abs() / amax.repeat_interleave(32, 1)
    # e4m3: 3 mantissa bits (half an ulp of the top binade = 1/16 of the block maximum) and, per the OCP MX rule
    # scale = 2^(floor(log2 amax) - 8), block maxima that land in (448, 512) saturate to 448 (at most 1/8 off)
    assert rel.max() < 0.15 and rel.mean() < 0.01


def test_fp8_linear_tracks_bf16():
    from nanonemo_b200 import fp8
    from nanonemo_b200.ops.gemm import linear_sm100

    torch.manual_seed(1)
    x = torch.randn(256, 768, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(1280, 768, device="cuda") * 0.02).requires_grad_()
    g = torch.randn(256, 1280, device="cuda", dtype=torch.bfloat16)
    with fp8.fp8_context("delayed")():
        y8 = fp8.linear_mxfp8(x, w)
    y8.backward(g)
    gx8, gw8 = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    y16 = linear_sm100(x, w)
    y16.backward(g)
    for a, b in ((y8, y16), (gx8, x.grad), (gw8, w.grad)):
        err = (a.float() - b.float()).norm() / b.float().norm()
        assert err < 6e-2, err
    assert fp8.linear_mxfp8(x, w).sub(y16).abs().max() == 0  # outside the context: the plain 16-bit GEMM


def test_fp8_precision_trains(tmp_path):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.train.config import TrainConfig
    from nanonemo_b200.train.trainer import train

    losses = {}
    for prec, lin in (("bf16", "sm100"), ("fp8", "mxfp8")):
        mc = ModelConfig.sm100(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, d_ff=512, max_seq_len=256, linear_impl=lin)
        tc = TrainConfig(data_dir="synthetic", out_dir=str(tmp_path / prec), seq_len=256, micro_batch=8, global_batch_tokens=2048,
                         total_tokens=2048 * 10, peak_lr=1e-3, precision=prec, eval_every=100, eval_batches=1)
        losses[prec] = [r["loss"] for r in train(mc, tc, device="cuda:0") if "loss" in r]
    assert losses["fp8"] == pytest.approx(losses["bf16"], abs=2e-2)
