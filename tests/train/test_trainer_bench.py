"""Trainer behaviour on CPU: accumulation, learning, records, checkpoint/resume, benchmark structure, W&B mapping."""

import json

import numpy as np
import pytest
import torch

from nanonemo_b200.data.shard import write_shard
from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.train.config import TrainConfig
from nanonemo_b200.train.trainer import train

TINY = ModelConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=32)


def pattern_dataset(root, n=40000, period=7):
    root.mkdir(parents=True, exist_ok=True)
    toks = (np.arange(n) % period) * 3 + 1  # a learnable repeating pattern
    splits = {}
    for split, t in (("train", toks), ("val", toks[:4000])):
        info = write_shard(root / f"{split}.bin", t, "gpt2")
        splits[split] = {"n_tokens": len(t), "shards": [{"path": f"{split}.bin", **info}]}
    (root / "manifest.json").write_text(json.dumps({"tokenizer": "gpt2", "splits": splits}))
    return str(root)


def base_cfg(tmp_path, **kw):
    d = dict(data_dir=pattern_dataset(tmp_path / "data"), out_dir=str(tmp_path / "run"), seq_len=32, micro_batch=4,
             global_batch_tokens=256, total_tokens=256 * 30, peak_lr=3e-3, eval_every=10, eval_batches=2, ckpt_async=False)
    d.update(kw)
    return TrainConfig(**d)


def test_trainer_learns_and_persists_records(tmp_path):
    cfg = base_cfg(tmp_path)
    history = train(TINY, cfg, device="cpu")
    losses = [r["loss"] for r in history if "loss" in r]
    assert len(losses) == 30 and losses[-1] < 0.5 * losses[0]
    assert history[0]["event"] == "start" and history[0]["grad_accum"] == 2 and history[0]["params"] > 0
    vals = [r["val_loss"] for r in history if "val_loss" in r]
    assert len(vals) == 3 and vals[-1] < vals[0]
    lines = [json.loads(l) for l in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines()]
    assert lines == json.loads(json.dumps(history))
    assert (tmp_path / "run" / "config.yaml").exists()
    for r in history:
        if "loss" in r:
            assert {"step", "lr", "grad_norm", "tokens", "tokens_per_s"} <= set(r)


def test_grad_accumulation_equals_one_big_batch(tmp_path):
    a = train(TINY, base_cfg(tmp_path / "a", micro_batch=8, total_tokens=256 * 4), device="cpu")
    b = train(TINY, base_cfg(tmp_path / "b", micro_batch=2, total_tokens=256 * 4), device="cpu")
    la, lb = [r["loss"] for r in a if "loss" in r], [r["loss"] for r in b if "loss" in r]
    assert la == pytest.approx(lb, rel=1e-4, abs=1e-5)
    ga, gb = [r["grad_norm"] for r in a if "loss" in r], [r["grad_norm"] for r in b if "loss" in r]
    assert ga == pytest.approx(gb, rel=1e-3)


def test_stop_and_resume_equals_uninterrupted(tmp_path):
    full = train(TINY, base_cfg(tmp_path / "full", total_tokens=256 * 8), device="cpu")
    part = train(TINY, base_cfg(tmp_path / "part", total_tokens=256 * 8, max_steps=3), device="cpu")
    assert part[-1]["event"] == "stopped" and part[-1]["reason"] == "max_steps"
    ckpt = tmp_path / "part" / "run" / "ckpt"
    assert (ckpt / "latest").read_text() == "step_000002" and (ckpt / "step_000002" / "trainer.json").exists()
    rest = train(TINY, base_cfg(tmp_path / "part", total_tokens=256 * 8, resume_from=str(ckpt)), device="cpu")
    assert rest[0]["start_step"] == 3 and rest[0]["resumed_from"].endswith("step_000002")
    lf = [r["loss"] for r in full if "loss" in r]
    lr_ = [r["loss"] for r in part + rest if "loss" in r]
    assert lf == pytest.approx(lr_, rel=1e-5)
    lines = (tmp_path / "part" / "run" / "metrics.jsonl").read_text().splitlines()
    assert sum('"loss"' in l and "val" not in l for l in lines) == 8  # appended, not truncated


def test_checkpoints_are_pruned_and_latest_points_to_complete_one(tmp_path):
    from nanonemo_b200.train.checkpoint import find_latest

    train(TINY, base_cfg(tmp_path, total_tokens=256 * 7, ckpt_every=2), device="cpu")
    root = tmp_path / "run" / "ckpt"
    kept = sorted(p.name for p in root.glob("step_*"))
    assert kept == ["step_000005", "step_000006"]
    assert find_latest(root).name == "step_000006" and find_latest(root / "step_000005").name == "step_000005"
    (root / "latest").write_text("step_000099")  # points at something that was never completed
    assert find_latest(root) is None
    assert find_latest(tmp_path / "nowhere") is None


def test_parallel_needs_torchrun(tmp_path):
    with pytest.raises(ValueError, match="torchrun"):
        train(TINY, base_cfg(tmp_path, parallel="ddp"), device="cpu")


def test_benchmark_structure_on_cpu(tmp_path):
    from nanonemo_b200.train.bench import benchmark

    r = benchmark(TINY, base_cfg(tmp_path), steps=3, trials=2, warmup_steps=1, device="cpu")
    json.dumps(r)
    assert r["bench"]["grad_accum"] == 2 and len(r["trials"]) == 2 and len(r["trials"][0]["step_ms"]) == 3
    t = r["trials"][0]
    assert t["tokens_per_s"] == pytest.approx(3 * 256 / (sum(t["step_ms"]) / 1e3))
    assert r["tokens_per_s"]["min"] <= r["tokens_per_s"]["median"] <= r["tokens_per_s"]["max"]
    assert r["flops_per_token"] > 0 and r["mfu"] is None and r["params"] > 0


def test_wandb_mapping():
    from nanonemo_b200.train.wandb_sink import to_wandb

    out = to_wandb({"step": 3, "loss": 1.0, "lr": 0.1, "tokens_per_s": 5.0, "mfu": 0.3, "event": "x"})
    assert out == {"train/loss": 1.0, "train/lr": 0.1, "perf/tokens_per_s": 5.0, "perf/mfu": 0.3}
    assert to_wandb({"step": 1, "val_loss": 2.0}) == {"val/loss": 2.0}


def test_train_step_raises_when_a_kernel_status_word_is_set(tmp_path):
    """The step's single device -> host read carries the kernels' status flag: a non-zero word (a bounded wait inside a
    collective or a tensor-core pipeline ran out) makes the step raise instead of training on with skipped work."""
    from nanonemo_b200 import parallel
    from nanonemo_b200.data.loader import TokenLoader
    from nanonemo_b200.train.optim import build_optimizer
    from nanonemo_b200.train.trainer import build_parallel, train_step

    cfg = TrainConfig(data_dir="synthetic", out_dir=str(tmp_path), seq_len=32, micro_batch=2, global_batch_tokens=64, total_tokens=640)
    tiny = ModelConfig(n_layers=1, d_model=32, n_heads=2, n_kv_heads=1, d_ff=64, vocab_size=50304, max_seq_len=32)
    strategy = build_parallel(tiny, cfg, parallel.Dist(device="cpu"))
    opt = build_optimizer(strategy.model, 1e-3, 0.1, store=strategy.store)
    loader = TokenLoader("synthetic", "train", 32, 2, device="cpu")
    loss, norm = train_step(strategy, opt, loader, 1, 1.0)
    assert loss == loss and norm > 0  # nothing to watch on the CPU: plain (loss, norm)
    word = torch.zeros(8, dtype=torch.int32)
    strategy.status_words = lambda: [word]
    assert len(train_step(strategy, opt, loader, 1, 1.0)) == 2  # a clear word changes nothing
    out = train_step(strategy, opt, loader, 1, 1.0, host_sync=False)
    assert out.shape == (3,) and out[2].item() == 0
    word[0] = 11  # what a collective kernel records when its wait for a peer gives up
    with pytest.raises(RuntimeError, match="bounded wait"):
        train_step(strategy, opt, loader, 1, 1.0)
    assert train_step(strategy, opt, loader, 1, 1.0, host_sync=False)[2].item() == 1
