"""Checkpoints are interchangeable with the reference's: same DCP keys, per-projection weights, optimizer state layout.

The reference package (unmodified, installed under baseline/_ref) writes a checkpoint with its own ``Checkpointer`` and this
framework resumes from it; then this framework writes one and the reference's own ``load`` reads it back. Skipped when the
reference package is not installed."""

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[2]
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "nanonemo" / "train" / "checkpoint.py").exists(), reason="reference package not installed")

SHAPE = dict(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=32)
TRAINER = {"step": 3, "micro_step": 4, "scaler": None, "world": 1, "dp_world": 1, "parallel": "none"}


@pytest.fixture
def ref():
    sys.path.insert(0, str(REF))
    try:
        from nanonemo.model.config import ModelConfig
        from nanonemo.model.model import NanoNemo
        from nanonemo.train import checkpoint
        from nanonemo.train.optim import build_optimizer

        yield type("Ref", (), dict(ModelConfig=ModelConfig, NanoNemo=NanoNemo, checkpoint=checkpoint, build_optimizer=staticmethod(build_optimizer)))
    finally:
        sys.path.remove(str(REF))


def _one_step(model, opt, seed):
    torch.manual_seed(seed)
    idx = torch.randint(0, 512, (2, 33))
    _, loss = model(idx[:, :-1], idx[:, 1:])
    loss.backward()
    opt.step()
    opt.zero_grad()


def _fused_views(ours):
    """name -> tensor under the reference's parameter names, from this framework's fused parameters."""
    out = {}
    for n, p in ours.named_parameters():
        if n.endswith("attn.wqkv.weight"):
            stem = n[: -len("wqkv.weight")]
            cfg = ours.cfg
            q, kv = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
            out[stem + "wq.weight"], out[stem + "wk.weight"], out[stem + "wv.weight"] = p[:q], p[q:q + kv], p[q + kv:]
        elif n.endswith("mlp.w_gu.weight"):
            stem = n[: -len("w_gu.weight")]
            out[stem + "w_gate.weight"], out[stem + "w_up.weight"] = p[: p.shape[0] // 2], p[p.shape[0] // 2:]
        else:
            out[n] = p
    return out


def test_resume_from_a_checkpoint_written_by_the_reference(tmp_path, ref):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.models.model import NanoNemo
    from nanonemo_b200.train import checkpoint
    from nanonemo_b200.train.optim import build_optimizer

    torch.manual_seed(0)
    theirs = ref.NanoNemo(ref.ModelConfig(**SHAPE))
    their_opt = ref.build_optimizer(theirs, 1e-3, 0.1)
    _one_step(theirs, their_opt, 1)
    _one_step(theirs, their_opt, 2)
    ref.checkpoint.Checkpointer(tmp_path, True, use_async=False).save(3, theirs, their_opt, TRAINER)

    ours = NanoNemo(ModelConfig(**SHAPE))
    opt = build_optimizer(ours, 1e-3, 0.1)
    state = checkpoint.load(checkpoint.find_latest(tmp_path), ours, opt)
    assert state["step"] == 3 and state["micro_step"] == 4
    mine = _fused_views(ours)
    for n, p in theirs.named_parameters():
        assert torch.equal(mine[n], p), n
        st = their_opt.state[p]
        mine_state = {k: v for k, v in _fused_views_of_state(ours, opt, "exp_avg").items()}
        assert torch.equal(mine_state[n], st["exp_avg"]), n
    assert ours.lm_head.weight is ours.tok_emb.weight
    assert all(float(st["step"]) == 2 for st in opt.state.values())
    # and training goes on identically from there
    _one_step(theirs, their_opt, 5)
    _one_step(ours, opt, 5)
    mine = _fused_views(ours)
    for n, p in theirs.named_parameters():
        assert torch.allclose(mine[n], p, atol=1e-6), n


def _fused_views_of_state(ours, opt, key):
    shadow = type(ours)(ours.cfg)
    with torch.no_grad():
        for (n, p), q in zip(ours.named_parameters(), shadow.parameters()):
            q.copy_(opt.state[p][key])
    return _fused_views(shadow)


def test_the_reference_reads_a_checkpoint_written_here(tmp_path, ref):
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.models.model import NanoNemo
    from nanonemo_b200.train import checkpoint
    from nanonemo_b200.train.optim import build_optimizer

    torch.manual_seed(0)
    ours = NanoNemo(ModelConfig(**SHAPE))
    opt = build_optimizer(ours, 1e-3, 0.1)
    _one_step(ours, opt, 1)
    checkpoint.Checkpointer(tmp_path, True, use_async=False).save(7, ours, opt, dict(TRAINER, step=7))

    theirs = ref.NanoNemo(ref.ModelConfig(**SHAPE))
    their_opt = ref.build_optimizer(theirs, 1e-3, 0.1)
    state = ref.checkpoint.load(ref.checkpoint.find_latest(tmp_path), theirs, their_opt)
    assert state["step"] == 7
    mine, mine_avg = _fused_views(ours), _fused_views_of_state(ours, opt, "exp_avg_sq")
    for n, p in theirs.named_parameters():
        assert torch.equal(mine[n], p), n
        assert torch.equal(mine_avg[n], their_opt.state[p]["exp_avg_sq"]), n
        assert float(their_opt.state[p]["step"]) == 1
    _one_step(theirs, their_opt, 5)
    _one_step(ours, opt, 5)
    mine = _fused_views(ours)
    for n, p in theirs.named_parameters():
        assert torch.allclose(mine[n], p, atol=1e-6), n
