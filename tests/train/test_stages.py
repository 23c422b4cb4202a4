"""The optimisation ladder (configs/stages): structure on the CPU, parity between neighbouring stages on a GPU.

Structure: every stage file differs from the previous one by the setting its name announces, every ablation differs from
S4 by one. Parity (GPU): stages that only change HOW something is computed must train like the stage before them — the
memory-efficient attention backend vs the math one, 16-bit autocast vs fp32 over 40 steps, the micro-batch replayed from a
CUDA graph vs launched eagerly, the hand-written kernel stack vs the PyTorch operators — and every fp16 stage of the ladder
must actually run in fp16 (loss scaling, the kernels' fp16 paths) rather than only after an override to bf16.
Mirrors the reference's tests/train/test_stages.py:54-125."""

from pathlib import Path

import pytest
import torch

from nanonemo_b200.train.config import load_config

CONFIGS = Path(__file__).resolve().parents[2] / "configs"
SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, d_ff=512, vocab_size=50304, max_seq_len=256)


def _diff(a, b):
    (ma, ta), (mb, tb) = a, b
    return [k for k in vars(ma) if getattr(ma, k) != getattr(mb, k)] + [k for k in vars(ta) if getattr(ta, k) != getattr(tb, k)]


def test_each_stage_changes_the_one_setting_it_names():
    names = sorted(p.name for p in (CONFIGS / "stages").glob("s*.yaml"))
    assert [n.split("_")[0] for n in names] == [f"s{i}" for i in range(9)]
    stages = [load_config(CONFIGS / "stages" / n) for n in names]
    changed = [sorted(_diff(a, b)) for a, b in zip(stages, stages[1:])]
    assert changed == [["precision"], ["attn_backend"], ["compile"], ["compile"], ["norm_kernel", "rope_kernel", "swiglu_kernel"],
                       ["norm_kernel"], ["attn_kernel"], ["loss_kernel"]]
    s4 = stages[4]
    for f in (CONFIGS / "ablations").glob("*.yaml"):
        assert len(_diff(s4, load_config(f))) == 1, f.name


def _train(tmp_path, name, model_kw, steps=12, **train_kw):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.train.config import TrainConfig
    from nanonemo_b200.train.trainer import train

    kw = dict(data_dir="synthetic", out_dir=str(tmp_path / name), seq_len=256, micro_batch=4, global_batch_tokens=2048,
              total_tokens=2048 * steps, peak_lr=1e-3, eval_every=10**6, eval_batches=1)
    kw.update(train_kw)
    return [r["loss"] for r in train(ModelConfig(**{**SMALL, **model_kw}), TrainConfig(**kw), device="cuda:0") if "loss" in r]


@pytest.mark.gpu
def test_memory_efficient_attention_trains_like_math_attention(tmp_path):
    a = _train(tmp_path, "math", dict(attn_backend="math"), precision="bf16")
    b = _train(tmp_path, "mem", dict(attn_backend="mem_efficient"), precision="bf16")
    assert b == pytest.approx(a, rel=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["fp16", "bf16"])
def test_autocast_tracks_fp32_over_40_steps(tmp_path, precision):
    ref = _train(tmp_path, "fp32", dict(attn_backend="mem_efficient"), steps=40, precision="fp32")
    amp = _train(tmp_path, precision, dict(attn_backend="mem_efficient"), steps=40, precision=precision)
    assert len(amp) == 40 and amp == pytest.approx(ref, rel=2e-2)


@pytest.mark.gpu
def test_kernel_stack_tracks_the_pytorch_operators(tmp_path):
    from nanonemo_b200.models.config import ModelConfig

    torch_path = _train(tmp_path, "torch", dict(attn_backend="mem_efficient"), precision="bf16")
    kernels = {k: getattr(ModelConfig.sm100(), k) for k in ("norm_kernel", "swiglu_kernel", "rope_kernel", "attn_kernel", "loss_kernel",
                                                            "linear_impl", "embed_kernel", "attn_backend")}
    sm100 = _train(tmp_path, "sm100", kernels, precision="bf16")
    graph = _train(tmp_path, "graph", kernels, precision="bf16", cuda_graph=True)
    assert sm100 == pytest.approx(torch_path, abs=2e-2)
    assert graph == pytest.approx(sm100, abs=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("stage", ["s1_fp16", "s5_triton", "s7_cuda_attn", "s8_fused_ce"])
def test_fp16_stages_run_in_fp16(tmp_path, stage):
    """The stage files as written (precision fp16, loss scaling), shrunk to a small model and a few steps."""
    from dataclasses import replace

    from nanonemo_b200.train.trainer import train

    model_cfg, cfg = load_config(CONFIGS / "stages" / f"{stage}.yaml")
    assert cfg.precision == "fp16"
    model_cfg = replace(model_cfg, **SMALL)
    cfg = replace(cfg, data_dir="synthetic", out_dir=str(tmp_path / stage), seq_len=256, micro_batch=2, global_batch_tokens=1024,
                  total_tokens=1024 * 6, eval_every=10**6, compile=None)
    recs = [r for r in train(model_cfg, cfg, device="cuda:0") if "loss" in r]
    assert len(recs) == 6 and all(r["loss"] == r["loss"] for r in recs) and recs[-1]["loss"] < 12
    assert all(r.get("loss_scale") for r in recs)
