"""Run configuration (YAML, validation, overrides), optimizer groups, LR schedule, stage ladder."""

import math
from pathlib import Path

import pytest
import torch
import yaml

from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.model import NanoNemo
from nanonemo_b200.train.config import TrainConfig, apply_overrides, dump_config, load_config
from nanonemo_b200.train.optim import build_optimizer, lr_at, param_groups

CONFIGS = Path(__file__).resolve().parents[2] / "configs"


def test_every_config_loads():
    files = sorted(CONFIGS.rglob("*.yaml"))
    assert len(files) >= 33
    for f in files:
        load_config(f)


def test_typos_and_bad_values_are_rejected(tmp_path):
    (tmp_path / "a.yaml").write_text("train: {micro_batchh: 4}")
    with pytest.raises(ValueError, match="micro_batchh"):
        load_config(tmp_path / "a.yaml")
    (tmp_path / "b.yaml").write_text("optimizer: {lr: 1}")
    with pytest.raises(ValueError, match="sections"):
        load_config(tmp_path / "b.yaml")
    for bad in (dict(precision="fp64"), dict(parallel="pp"), dict(compile="fast"), dict(fp8_recipe="x"),
                dict(parallel="ddp", compile="reduce-overhead"), dict(fsdp_compile_blocks=True),
                dict(fsdp_param_dtype="int8"), dict(parallel="fsdp_tp")):
        with pytest.raises(ValueError):
            TrainConfig(**bad)


def test_round_trip_and_overrides(tmp_path):
    m, t = ModelConfig(norm_kernel="sm100"), TrainConfig(micro_batch=8, parallel="ddp")
    (tmp_path / "c.yaml").write_text(dump_config(m, t))
    assert load_config(tmp_path / "c.yaml") == (m, t)
    m2, t2 = apply_overrides(m, t, ["train.max_steps=7", "model.attn_kernel=sm100", "train.peak_lr=1.0e-3", "train.compile=null"])
    assert (t2.max_steps, m2.attn_kernel, t2.peak_lr, t2.compile) == (7, "sm100", 1e-3, None)
    with pytest.raises(ValueError):
        apply_overrides(m, t, ["train.nope=1"])
    with pytest.raises(ValueError):
        apply_overrides(m, t, ["max_steps=1"])


def test_derived_arithmetic():
    t = TrainConfig(seq_len=1024, micro_batch=4, global_batch_tokens=65536, total_tokens=65536 * 100, warmup_frac=0.02)
    assert t.grad_accum(1) == 16 and t.grad_accum(2) == 8 and t.total_steps == 100 and t.warmup_steps == 2
    with pytest.raises(ValueError, match="multiple"):
        t.grad_accum(3)
    assert not t.checkpointing and TrainConfig(max_steps=3).checkpointing and TrainConfig(ckpt_every=5).checkpointing


def _stage(name):
    return load_config(CONFIGS / "stages" / name)


def test_param_groups_and_hyperparameters():
    model = NanoNemo(ModelConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=32))
    decay, no_decay = param_groups(model, 0.1)
    assert decay["weight_decay"] == 0.1 and no_decay["weight_decay"] == 0.0
    assert all(p.dim() == 2 for p in decay["params"]) and len(decay["params"]) == 2 * 4
    assert any(p is model.tok_emb.weight for p in no_decay["params"]) and len(no_decay["params"]) == 1 + 2 * 2 + 1
    assert sum(p.numel() for g in (decay, no_decay) for p in g["params"]) == model.num_params()
    opt = build_optimizer(model, 3e-4, 0.1)
    assert opt.defaults["betas"] == (0.9, 0.95) and opt.defaults["eps"] == 1e-8


def test_lr_schedule_shape():
    peak, total, warm = 6e-4, 1000, 20
    lrs = [lr_at(s, peak, total, warm, 0.1) for s in range(total)]
    assert lrs[0] == pytest.approx(peak / warm) and lrs[warm - 1] == pytest.approx(peak)
    assert all(a < b for a, b in zip(lrs[:warm - 1], lrs[1:warm]))
    assert all(a >= b for a, b in zip(lrs[warm:], lrs[warm + 1:]))
    assert lrs[-1] == pytest.approx(0.1 * peak) and lr_at(5000, peak, total, warm, 0.1) == pytest.approx(0.1 * peak)
    mid = lr_at(warm + (total - 1 - warm) // 2, peak, total, warm, 0.1)
    assert mid == pytest.approx(peak * (0.1 + 0.9 * 0.5), rel=1e-2)


def test_flat_store_keeps_parameters_and_state_views():
    from nanonemo_b200.parallel.flat import FlatParams
    from nanonemo_b200.train.optim import FusedAdamW

    torch.manual_seed(0)
    cfg = ModelConfig(n_layers=1, d_model=32, n_heads=2, n_kv_heads=1, d_ff=64, vocab_size=128, max_seq_len=16)
    a, b = NanoNemo(cfg), NanoNemo(cfg)
    b.load_state_dict(a.state_dict())
    store = FlatParams(b, "cpu")
    opt_b = build_optimizer(b, 1e-2, 0.1, store=store)
    opt_a = build_optimizer(a, 1e-2, 0.1)
    assert isinstance(opt_b, FusedAdamW)
    idx = torch.randint(0, 128, (2, 9))
    for _ in range(3):
        for m, o in ((a, opt_a), (b, opt_b)):
            m(idx[:, :-1], idx[:, 1:])[1].backward()
            o.step()
        opt_a.zero_grad()
        store.zero_grad()
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        torch.testing.assert_close(pa, pb, msg=n)
        assert pb.data_ptr() >= store.master.data_ptr() and pb.grad.data_ptr() >= store.grad.data_ptr()
    st = opt_b.state[b.blocks[0].attn.wo.weight]
    assert st["exp_avg"].data_ptr() >= store.exp_avg.data_ptr() and float(st["step"]) == 3


def test_accepted_settings_without_effect_are_reported():
    from nanonemo_b200.train.config import TrainConfig

    assert TrainConfig().inert_settings() == []
    notes = TrainConfig(parallel="ddp", ddp_grad_as_bucket_view=True, compile="default").inert_settings()
    assert any(n.startswith("ddp_grad_as_bucket_view") for n in notes) and any(n.startswith("compile=default") for n in notes)
    assert TrainConfig(compile="default").inert_settings(model_uses_sm100=False) == []
    notes = TrainConfig(parallel="fsdp", fsdp_compile_blocks=True, precision="fp8").inert_settings()
    assert any(n.startswith("fsdp_compile_blocks") for n in notes) and any(n.startswith("fp8_recipe=delayed") for n in notes)
