"""Fused linear + cross-entropy, and whole-model parity of the sm100 path against the PyTorch path."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("N,D,V,chunk", [(512, 256, 1024, None), (1000, 768, 50304, 384), (130, 64, 520, 64)])
def test_linear_ce_loss_and_grads(N, D, V, chunk):
    from nanonemo_b200 import ops
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(N)
    x = (torch.randn(N, D, device=DEV) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, D, device=DEV) * 0.05).requires_grad_()
    t = torch.randint(0, V, (N,), device=DEV)
    loss = ops.linear_cross_entropy(x, w, t, chunk_rows=chunk)
    (loss * 3.0).backward()  # non-unit upstream gradient
    check_status()
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    ref = F.cross_entropy(xr @ wr.t(), t)
    (ref * 3.0).backward()
    torch.testing.assert_close(loss, ref, rtol=2e-3, atol=2e-3)
    for got, want in ((x.grad, xr.grad), (w.grad, wr.grad)):
        err = (got.float() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 1e-5, err


@pytest.mark.parametrize("world", [1, 2, 4])
def test_vocab_parallel_linear_ce_over_emulated_ranks(world):
    """Every 'rank' holds V/world rows of the head; the stats exchange is emulated by running the ranks' first halves,
    concatenating their stats, then running the second halves. Loss and gradients must equal the unsharded fp32 loss."""
    from nanonemo_b200.ops import linear_ce
    from nanonemo_b200.ops.gemm import check_status, gemm

    torch.manual_seed(world)
    N, D, V = 640, 128, 2048
    Vl = V // world
    x = (torch.randn(N, D, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(V, D, device=DEV) * 0.2).bfloat16()
    t = torch.randint(0, V, (N,), device=DEV)
    t[5] = -100  # ignored row
    logits = [gemm(x, w[r * Vl:(r + 1) * Vl].contiguous()) for r in range(world)]
    ref_logits = torch.cat([l.float() for l in logits], dim=1).requires_grad_()
    stats = [torch.empty(N, 4, device=DEV) for _ in range(world)]
    for r in range(world):
        linear_ce._ce_stats(logits[r], t, stats[r], r * Vl)
    stats_all = torch.cat(stats)
    losses = [torch.empty(N, device=DEV) for _ in range(world)]
    for r in range(world):
        linear_ce._ce_grad_vp(logits[r], t, stats_all, losses[r], r * Vl, V, world, 1.0 / N)
    check_status()
    ref_rows = F.cross_entropy(ref_logits, t, reduction="none", ignore_index=-100)
    (ref_rows.sum() / N).backward()
    for r in range(world):
        torch.testing.assert_close(losses[r], ref_rows.detach(), rtol=1e-4, atol=1e-4)
    got = torch.cat([l.float() for l in logits], dim=1)
    assert (got - ref_logits.grad).abs().max().item() <= 1e-2 * ref_logits.grad.abs().max().item() + 1e-7
    assert got[5].abs().max().item() == 0.0


def test_linear_ce_peak_memory_is_far_below_unfused():
    from nanonemo_b200 import ops

    N, D, V = 8192, 768, 50304
    x = torch.randn(N, D, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(V, D, device=DEV) * 0.02).requires_grad_()
    t = torch.randint(0, V, (N,), device=DEV)

    def peak(fn):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        fn().backward()
        torch.cuda.synchronize()
        x.grad = w.grad = None
        return torch.cuda.max_memory_allocated() - base

    fused = peak(lambda: ops.linear_cross_entropy(x, w, t, chunk_rows=2048))
    unfused = peak(lambda: F.cross_entropy(F.linear(x, w.bfloat16()).float(), t))
    assert fused < 0.6 * unfused, (fused, unfused)


SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, d_ff=512, vocab_size=50304, max_seq_len=256)
SWITCHES = ["norm_kernel", "swiglu_kernel", "rope_kernel", "attn_kernel", "loss_kernel", "linear_impl", "embed_kernel"]


def _run(cfg_kw, idx):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.models.model import NanoNemo

    torch.manual_seed(0)
    model = NanoNemo(ModelConfig(**SMALL, attn_backend="math", **cfg_kw)).to(DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        _, loss = model(idx[:, :-1], idx[:, 1:])
    loss.backward()
    return loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("switch", SWITCHES + ["all"])
def test_model_with_each_kernel_matches_torch_path(switch):
    from nanonemo_b200.ops.gemm import check_status

    torch.manual_seed(1)
    idx = torch.randint(0, 50257, (4, 257), device=DEV)
    ref_loss, ref_grads = _run({}, idx)
    kw = {s: "sm100" for s in SWITCHES} if switch == "all" else {switch: "sm100"}
    loss, grads = _run(kw, idx)
    check_status()
    assert loss == pytest.approx(ref_loss, abs=2e-2)
    for n, g in grads.items():
        denom = ref_grads[n].norm().item() + 1e-8
        assert (g - ref_grads[n]).norm().item() / denom < 5e-2, (switch, n)


def test_sm100_training_tracks_torch_training(tmp_path):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.train.config import TrainConfig
    from nanonemo_b200.train.trainer import train

    out = {}
    for name, mc in (("torch", ModelConfig(**SMALL, attn_backend="mem_efficient")), ("sm100", ModelConfig.sm100(**SMALL))):
        tc = TrainConfig(data_dir="synthetic", out_dir=str(tmp_path / name), seq_len=256, micro_batch=4, global_batch_tokens=2048,
                         total_tokens=2048 * 12, peak_lr=1e-3, precision="bf16", eval_every=100, eval_batches=1)
        out[name] = [r["loss"] for r in train(mc, tc, device="cuda:0") if "loss" in r]
    assert out["sm100"] == pytest.approx(out["torch"], abs=2e-2)  # uniform-random tokens: the loss itself stays near ln V


def test_cuda_graph_training_matches_eager(tmp_path):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.train.config import TrainConfig
    from nanonemo_b200.train.trainer import train

    out = {}
    for name, graph in (("eager", False), ("graph", True)):
        tc = TrainConfig(data_dir="synthetic", out_dir=str(tmp_path / name), seq_len=256, micro_batch=2, global_batch_tokens=1024,
                         total_tokens=1024 * 10, peak_lr=1e-3, precision="bf16", eval_every=100, eval_batches=1, cuda_graph=graph)
        out[name] = [r["loss"] for r in train(ModelConfig.sm100(**SMALL), tc, device="cuda:0") if "loss" in r]
    assert out["graph"] == pytest.approx(out["eager"], abs=2e-2)
