"""Real GPUs: every layout on the sm100 kernels with the fused NVLink collectives must track the single-GPU losses (bf16,
tolerance 2e-2). Two GPUs go through the real CLI under torch.distributed.run, layout by layout; 2, 4 and 8 GPUs run
``parity_worker.py`` once per world size (exact checks of the collective kernels, then all layouts in one process group)."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[2]
pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

CONFIG = """
model: {n_layers: 2, d_model: 256, n_heads: 4, n_kv_heads: 2, d_ff: 512, vocab_size: 50304, max_seq_len: 256,
        norm_kernel: sm100, swiglu_kernel: sm100, rope_kernel: sm100, attn_kernel: sm100, linear_impl: sm100,
        loss_kernel: LOSS, embed_kernel: EMBED, attn_backend: mem_efficient}
train: {data_dir: synthetic, out_dir: OUT, seq_len: 256, micro_batch: 4, global_batch_tokens: 2048, total_tokens: 16384,
        peak_lr: 1.0e-3, precision: bf16, eval_every: 100, eval_batches: 1, ckpt_async: false}
"""


def run(tmp_path, name, nproc, *overrides, loss="sm100", embed="sm100", port=29561):
    out = tmp_path / name
    cfg = tmp_path / f"{name}.yaml"
    cfg.write_text(CONFIG.replace("OUT", str(out)).replace("LOSS", loss).replace("EMBED", embed))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    base = [str(ROOT / "scripts" / "train.py"), "--config", str(cfg), "--set", *overrides]
    cmd = [sys.executable] + base if nproc == 1 else [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
        "--master-port", str(port)] + base
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    recs = [json.loads(l) for l in (out / "metrics.jsonl").read_text().splitlines()]
    return [x["loss"] for x in recs if "loss" in x]


@pytest.mark.parametrize("par,extra,loss,embed", [
    ("ddp", ("train.comm=fused",), "sm100", "sm100"),
    ("ddp", ("train.comm=nccl",), "sm100", "sm100"),
    ("fsdp", ("train.comm=fused", "train.fsdp_prefetch=true"), "sm100", "sm100"),
    ("fsdp", ("train.comm=nccl",), "sm100", "sm100"),
    ("tp", ("train.comm=nccl",), "torch", "torch"),
    ("tp", ("train.comm=fused",), "torch", "torch"),
    ("tp", ("train.comm=fused",), "sm100", "sm100"),  # vocabulary-parallel fused linear + cross-entropy kernels
], ids=["ddp_fused", "ddp_nccl", "fsdp_fused", "fsdp_nccl", "tp_nccl", "tp_fused", "tp_fused_loss"])
def test_two_gpus_track_one_gpu(tmp_path, par, extra, loss, embed):
    single = run(tmp_path, "one", 1, "train.parallel=none", loss=loss, embed=embed)
    multi = run(tmp_path, "two", 2, f"train.parallel={par}", *extra, loss=loss, embed=embed)
    assert len(single) == len(multi) == 8
    assert multi == pytest.approx(single, abs=2e-2), (single, multi)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_layouts_and_collectives_at_world_size(world):
    """Exact all-reduce / reduce-scatter / all-gather values and in-kernel gradient norm at this world size, then ddp, ddp replayed
    from a CUDA graph, fsdp, tp (rank pairs at 8: 4 KV heads) and the fsdp x tp mesh against a single-GPU run."""
    import torch

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
                        "127.0.0.1", "--master-port", str(29580 + world), str(ROOT / "tests" / "distributed" / "parity_worker.py")],
                       env=env, capture_output=True, text=True, timeout=900)
    print(r.stdout[-4000:])
    assert r.returncode == 0 and "PARITY_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
