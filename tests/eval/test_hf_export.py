"""HF-Llama export: identical logits, tied weights survive, checkpoints load through the exporter."""

import pytest
import torch

from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.model import NanoNemo

transformers = pytest.importorskip("transformers")

CFG = ModelConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=32)


def test_exported_model_has_identical_logits_and_stays_tied(tmp_path):
    from nanonemo_b200.eval.hf_export import export, to_hf

    torch.manual_seed(0)
    model = NanoNemo(CFG).eval()
    hf = to_hf(model)
    idx = torch.randint(0, 512, (2, 20))
    with torch.no_grad():
        ours, theirs = model(idx)[0], hf(idx).logits
    torch.testing.assert_close(ours, theirs, rtol=1e-4, atol=1e-4)
    assert hf.lm_head.weight.data_ptr() == hf.model.embed_tokens.weight.data_ptr()
    out = export(model, tmp_path / "hf", tokenizer=False)
    again = transformers.LlamaForCausalLM.from_pretrained(out)
    with torch.no_grad():
        torch.testing.assert_close(again(idx).logits, ours, rtol=1e-4, atol=1e-4)


def test_training_checkpoint_round_trips_through_load_checkpoint(tmp_path):
    from nanonemo_b200.eval.hf_export import load_checkpoint
    from nanonemo_b200.train.checkpoint import Checkpointer, find_latest
    from nanonemo_b200.train.optim import build_optimizer

    torch.manual_seed(1)
    model = NanoNemo(CFG)
    opt = build_optimizer(model, 1e-3)
    model(torch.randint(0, 512, (2, 9)), torch.randint(0, 512, (2, 9)))[1].backward()
    opt.step()
    ck = Checkpointer(tmp_path / "ckpt", main=True, use_async=False)
    ck.save(0, model, opt, {"step": 0, "micro_step": 1})
    loaded = load_checkpoint(find_latest(tmp_path / "ckpt"), CFG)
    for (n, a), (_, b) in zip(model.named_parameters(), loaded.named_parameters()):
        assert torch.equal(a, b), n
    assert loaded.lm_head.weight is loaded.tok_emb.weight
