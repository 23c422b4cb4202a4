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


def _dequant_chunked(q, sf):
    from nanonemo_b200 import fp8

    return fp8.dequantize(q, fp8.scales_to_plain(sf, q.shape[0], q.shape[1]).contiguous())


def test_tile_quantiser_matches_the_plain_quantiser_both_ways():
    from nanonemo_b200 import fp8

    torch.manual_seed(2)
    x = (torch.randn(384, 256, device="cuda") * torch.logspace(-2, 2, 256, device="cuda")).bfloat16()
    q, sf, qt, sft = fp8.quantize_mx(x, True, True)
    q_ref, s_ref = fp8.quantize(x)
    assert torch.equal(q, q_ref) and torch.equal(fp8.scales_to_plain(sf, 384, 256), s_ref)
    qt_ref, st_ref = fp8.quantize(x.t().contiguous())
    assert torch.equal(qt, qt_ref) and torch.equal(fp8.scales_to_plain(sft, 256, 384), st_ref)
    only_t = fp8.quantize_mx(x, False, True)
    assert only_t[0] is None and torch.equal(only_t[2], qt_ref)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1024, 2304, 768), (512, 768, 2048)])
def test_block_scaled_gemm_matches_fp32_product_of_the_quantised_values(M, N, K):
    """The tensor-core path must multiply exactly the MXFP8 values: compare with an fp32 matmul of the dequantised operands."""
    from nanonemo_b200 import fp8
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(M + N + K)
    # per-column magnitudes spread over several binades so that a wrong scale (row, k-block or byte) cannot go unnoticed
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 1, K, device="cuda")[torch.randperm(K, device="cuda")]).bfloat16()
    b = (torch.randn(N, K, device="cuda") * torch.logspace(-1, 1, N, device="cuda").unsqueeze(1)).bfloat16()
    aq, asf, _, _ = fp8.quantize_mx(a)
    bq, bsf, _, _ = fp8.quantize_mx(b)
    want = _dequant_chunked(aq, asf) @ _dequant_chunked(bq, bsf).t()
    got32 = fp8.gemm_mxfp8(aq, asf, bq, bsf, out_dtype=torch.float32)
    got16 = fp8.gemm_mxfp8(aq, asf, bq, bsf)
    check_status()
    scale = want.abs().max().item()
    assert (got32 - want).abs().max().item() <= 2e-5 * scale * (K / 128) ** 0.5 + 1e-6
    assert (got16.float() - want).abs().max().item() <= 1e-2 * scale
    acc = torch.ones(M, N, device="cuda")
    fp8.gemm_mxfp8(aq, asf, bq, bsf, out=acc, accumulate=True, k_splits=min(2, K // 128))
    check_status()
    assert (acc - 1.0 - want).abs().max().item() <= 2e-5 * scale * (K / 128) ** 0.5 + 1e-5


def test_fp8_linear_tensor_core_path_equals_the_emulation(monkeypatch):
    from nanonemo_b200 import fp8

    torch.manual_seed(3)
    x = torch.randn(512, 768, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(1280, 768, device="cuda") * 0.02).requires_grad_()
    g = torch.randn(512, 1280, device="cuda", dtype=torch.bfloat16)
    out = {}
    for emulate in ("0", "1"):
        monkeypatch.setenv("NANONEMO_FP8_EMULATE", emulate)
        x.grad = w.grad = None
        with fp8.fp8_context("mxfp8")():
            y = fp8.linear_mxfp8(x, w)
        y.backward(g)
        out[emulate] = (y.detach().float(), x.grad.float().clone(), w.grad.float().clone())
    for real, emu in zip(out["0"], out["1"]):
        # same quantised values; only the accumulation order and the output rounding differ
        assert (real - emu).abs().max().item() <= 1e-2 * emu.abs().max().item()
