"""Multi-process parity through the real CLI: 2 gloo ranks on CPU must reproduce the single-process
losses for every layout, resume must equal an uninterrupted run, and a checkpoint written under one
layout must resume under another (FSDP on 2 ranks -> 1 process; DDP 2 ranks -> TP 2 ranks)."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[2]
pytestmark = pytest.mark.distributed

CONFIG = """
model: {n_layers: 2, d_model: 128, n_heads: 4, n_kv_heads: 2, d_ff: 384, vocab_size: 50304, max_seq_len: 128}
train: {data_dir: synthetic, out_dir: OUT, seq_len: 128, micro_batch: 4, global_batch_tokens: 1024, total_tokens: 6144,
        peak_lr: 3.0e-4, eval_every: 100, eval_batches: 1, ckpt_async: false}
"""


def run(tmp_path, name, nproc, *overrides, port=29541):
    out = tmp_path / name
    cfg = tmp_path / f"{name}.yaml"
    cfg.write_text(CONFIG.replace("OUT", str(out)))
    env = dict(os.environ, NANONEMO_DEVICE="cpu", OMP_NUM_THREADS="2")
    cmd = [sys.executable, str(ROOT / "scripts" / "train.py"), "--config", str(cfg), "--set", *overrides]
    if nproc > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port)] + cmd[1:]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    recs = [json.loads(l) for l in (out / "metrics.jsonl").read_text().splitlines()]
    return [x["loss"] for x in recs if "loss" in x], out


@pytest.fixture(scope="module")
def single(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("single")
    losses, _ = run(tmp, "single", 1, "train.parallel=none")
    assert len(losses) == 6
    return losses


@pytest.mark.parametrize("overrides", [
    ("train.parallel=ddp",),
    ("train.parallel=ddp", "train.ddp_bucket_mb=0.5", "train.ddp_grad_as_bucket_view=true"),
    ("train.parallel=fsdp",),
    ("train.parallel=fsdp", "train.fsdp_prefetch=true", "train.fsdp_reshard_after_forward=false"),
    ("train.parallel=tp",),
], ids=["ddp", "ddp_small_buckets", "fsdp", "fsdp_prefetch", "tp"])
def test_two_ranks_match_one_process(tmp_path, single, overrides):
    losses, _ = run(tmp_path, "par", 2, *overrides)
    assert losses == pytest.approx(single, abs=1e-4)


def test_grad_accumulation_under_ddp(tmp_path, single):
    losses, _ = run(tmp_path, "acc", 2, "train.parallel=ddp", "train.micro_batch=2")
    assert losses == pytest.approx(single, abs=1e-4)


@pytest.mark.parametrize("par", ["ddp", "fsdp", "tp"])
def test_stop_and_resume_matches_uninterrupted(tmp_path, single, par):
    first, out = run(tmp_path, "r", 2, f"train.parallel={par}", "train.max_steps=3")
    both, _ = run(tmp_path, "r", 2, f"train.parallel={par}", f"train.resume_from={out / 'ckpt'}")
    assert len(first) == 3 and both == pytest.approx(single, abs=1e-4)  # the resumed run appends to the same metrics file


def test_fsdp_checkpoint_resumes_in_one_process(tmp_path, single):
    first, out = run(tmp_path, "a", 2, "train.parallel=fsdp", "train.max_steps=3")
    (tmp_path / "b").mkdir()
    rest, _ = run(tmp_path, "b", 1, "train.parallel=none", f"train.resume_from={out / 'ckpt'}")
    assert first + rest == pytest.approx(single, abs=1e-4)


def test_ddp_checkpoint_resumes_under_tp(tmp_path, single):
    first, out = run(tmp_path, "a", 2, "train.parallel=ddp", "train.max_steps=3")
    rest, _ = run(tmp_path, "b", 2, "train.parallel=tp", f"train.resume_from={out / 'ckpt'}")
    assert first + rest == pytest.approx(single, abs=1e-4)


def test_2d_mesh_fsdp_x_tp_matches_one_process_and_resumes_elsewhere(tmp_path, single):
    """4 ranks = 2 data-parallel (fully sharded) x 2 tensor-parallel; then its checkpoint resumes under DDP on 2 ranks."""
    losses, _ = run(tmp_path, "mesh", 4, "train.tp_size=2", "train.parallel=fsdp_tp")
    assert losses == pytest.approx(single, abs=1e-4)
    first, out = run(tmp_path, "a", 4, "train.tp_size=2", "train.parallel=fsdp_tp", "train.max_steps=3")
    rest, _ = run(tmp_path, "b", 2, "train.parallel=ddp", f"train.resume_from={out / 'ckpt'}")
    assert first + rest == pytest.approx(single, abs=1e-4)


def test_a_rank_that_never_joins_times_out_on_the_host(tmp_path):
    """Failure detection without touching a GPU: one of two gloo ranks exits before the rendezvous
    completes its first collective; the survivor's collective must end with an error within the
    process-group timeout instead of hanging."""
    script = tmp_path / "die.py"
    script.write_text(
        "import os, sys, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {str(ROOT)!r})\n"
        "from nanonemo_b200 import parallel\n"
        "d = parallel.init(timeout_s=5)\n"
        "if d.rank == 1:\n"
        "    os._exit(0)  # leaves between steps, nothing in flight\n"
        "try:\n"
        "    dist.all_reduce(torch.ones(1))\n"
        "    print('UNEXPECTED: collective completed')\n"
        "except Exception as e:\n"
        "    print('PEER LOST:', type(e).__name__)\n"
        "os._exit(0)\n")
    env = dict(os.environ, NANONEMO_DEVICE="cpu")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29547", str(script)], env=env, capture_output=True, text=True, timeout=120)
    assert "PEER LOST" in r.stdout + r.stderr, r.stdout[-1500:] + r.stderr[-1500:]


def test_tp_degree_beyond_the_kv_heads_uses_rank_pairs(tmp_path, single):
    """4 tensor-parallel ranks with 2 KV heads: the heads split 2 ways, the ranks of a pair split the query rows (the layout
    that serves TP=8 with 12 query / 4 KV heads). Losses must match one process, and the checkpoint — full tensors rebuilt
    from one copy per head group — must resume in a single process."""
    first, out = run(tmp_path, "pairs", 4, "train.parallel=tp", "train.max_steps=3", port=29547)
    assert first == pytest.approx(single[:3], abs=1e-4)
    (tmp_path / "b").mkdir()
    rest, _ = run(tmp_path, "b", 1, "train.parallel=none", f"train.resume_from={out / 'ckpt'}")
    assert first + rest == pytest.approx(single, abs=1e-4)


def test_attention_layout_and_pair_slices_without_processes():
    """Pure layout logic: which degrees are head-aligned, which use rank pairs, and that the pair layout's local slices are
    identical inside a pair and rebuild the full tensors when one copy per head group is concatenated."""
    import types

    import torch

    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.parallel.tp import attention_layout, tp_local_slice

    cfg = ModelConfig()  # 12 query / 4 KV heads
    assert [attention_layout(cfg, t) for t in (1, 2, 4, 8)] == [(1, 1), (2, 1), (4, 1), (4, 2)]
    with pytest.raises(ValueError):
        attention_layout(cfg, 3)
    with pytest.raises(ValueError):
        attention_layout(cfg, 16)
    hd, D = cfg.head_dim, cfg.d_model
    full_qkv = torch.arange((cfg.n_heads + 2 * cfg.n_kv_heads) * hd * 4, dtype=torch.float32).view(-1, 4)
    full_wo = torch.arange(D * cfg.n_heads * hd, dtype=torch.float32).view(D, cfg.n_heads * hd)
    ranks = [types.SimpleNamespace(rank=r, world=8, attn_rank=r // 2, attn_world=4, pair=2) for r in range(8)]
    qkv = [tp_local_slice("blocks.0.attn.wqkv.weight", full_qkv, tp, cfg) for tp in ranks]
    wo = [tp_local_slice("blocks.0.attn.wo.weight", full_wo, tp, cfg) for tp in ranks]
    for p in range(4):
        assert torch.equal(qkv[2 * p], qkv[2 * p + 1]) and torch.equal(wo[2 * p], wo[2 * p + 1])
    q, kv = cfg.n_heads // 4 * hd, cfg.n_kv_heads // 4 * hd
    parts = qkv[::2]
    rebuilt = torch.cat([x[:q] for x in parts] + [x[q:q + kv] for x in parts] + [x[q + kv:] for x in parts])
    assert torch.equal(rebuilt, full_qkv) and torch.equal(torch.cat(wo[::2], dim=1), full_wo)
    # the MLP stays split 8 ways
    full_down = torch.arange(D * cfg.d_ff, dtype=torch.float32).view(D, cfg.d_ff)
    assert tp_local_slice("blocks.0.mlp.w_down.weight", full_down, ranks[3], cfg).shape == (D, cfg.d_ff // 8)


def test_each_rank_saves_its_share_only():
    """A checkpoint save hands DCP 1 / world of the state per rank under every layout (row blocks as DTensor shards)."""
    env = dict(os.environ, NANONEMO_DEVICE="cpu", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29549", str(ROOT / "tests" / "distributed" / "ckpt_share_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "SHARE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
