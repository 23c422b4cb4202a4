"""Reference arm of bench.py: the UNMODIFIED reference package (installed into baseline/_ref with
``pip install --no-index --no-deps --target baseline/_ref <reference>``) run through its own public
entry point ``nanonemo.train.bench.benchmark`` and its stock code path (``precision: bf16``,
``compile: default``, ``attn_backend: mem_efficient``, torch DDP for N > 1) on the headline config.

Nothing of this framework's models, kernels or engine is on that path. What the harness provides
is environment only: a synthetic uniform-random dataset written in the reference's own shard
format, and a stand-in ``tiktoken`` module because the reference builds the GPT-2 encoder at
import time, which needs a network download this machine cannot make; the stand-in exposes the two
constants the reference reads (``n_vocab``, ``eot_token``) and is never asked to tokenise.
"""

import json
import os
import struct
import sys
import tempfile
import time
import types
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
REF = ROOT / "_ref"


def unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def _install_tiktoken_stub():
    try:
        import tiktoken

        tiktoken.get_encoding("gpt2")
        return
    except Exception:
        pass

    class _Enc:
        n_vocab, eot_token = 50257, 50256

        def encode_ordinary(self, text):
            raise RuntimeError("offline tiktoken stand-in: tokenising is not available")

        encode_ordinary_batch = decode = encode_ordinary

    stub = types.ModuleType("tiktoken")
    stub.get_encoding = lambda name: _Enc()
    sys.modules["tiktoken"] = stub


def _write_dataset(root: Path, train_tokens: int, val_tokens: int, seed: int = 0):
    """Uniform-random ids in [0, 50257) in the reference's shard format: 256-byte header
    ``<8sIQ32s`` (magic NNMOTOKS, version 1, token count, tokenizer name) + little-endian uint16 ids."""
    root.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    splits = {}
    for split, n in (("train", train_tokens), ("val", val_tokens)):
        ids = rng.integers(0, 50257, size=n, dtype=np.uint16)
        head = struct.pack("<8sIQ32s", b"NNMOTOKS", 1, n, b"gpt2").ljust(256, b"\0")
        name = f"{split}_000000.bin"
        with open(root / name, "wb") as f:
            f.write(head)
            f.write(ids.astype("<u2").tobytes())
        splits[split] = {"n_tokens": n, "shards": [{"path": name, "n_tokens": n}]}
    (root / "manifest.json").write_text(json.dumps({"tokenizer": "gpt2", "splits": splits}))


def main(a, headline_config=None):
    if not (REF / "nanonemo").is_dir():
        return unavailable("baseline/_ref is empty: install the reference package with pip --no-index --no-deps --target baseline/_ref <reference checkout>")
    import torch

    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    _install_tiktoken_stub()
    sys.path.insert(0, str(REF))
    try:
        from nanonemo import distributed
        from nanonemo.model.config import ModelConfig
        from nanonemo.train.bench import benchmark
        from nanonemo.train.config import TrainConfig
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference import failed: {type(e).__name__}: {e}")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE is {world}")
    micro, seq = a.micro_batch, 1024
    steps_total = a.warmup + a.steps + 2
    data_root = Path(tempfile.gettempdir()) / f"nanonemo_ref_data_{micro}_{world}_{steps_total}"
    if rank == 0 and not (data_root / "manifest.json").exists():
        _write_dataset(data_root, train_tokens=micro * seq * world * steps_total + 1 + seq, val_tokens=4 * micro * seq + 1)
    if world > 1:
        d = distributed.init()
        torch.distributed.barrier()
    model_cfg = ModelConfig(attn_backend="mem_efficient")
    par = getattr(a, "parallel", "ddp") if world > 1 else "none"
    dp = 1 if par == "tp" else world  # the reference's TP uses the whole world as one replica
    cfg = TrainConfig(data_dir=str(data_root), out_dir=str(data_root / "run"), seq_len=seq, micro_batch=micro,
                      global_batch_tokens=micro * seq * dp, precision="bf16", compile="default", parallel=par,
                      fsdp_prefetch=(par == "fsdp"))
    t0 = time.perf_counter()
    try:
        r = benchmark(model_cfg, cfg, steps=a.steps, trials=1, warmup_steps=a.warmup)
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference benchmark() raised {type(e).__name__}: {str(e)[:300]}")
    wall = time.perf_counter() - t0
    step_ms = r["trials"][0]["step_ms"]  # this rank's CUDA-event time of every optimizer step
    t = torch.tensor([sum(step_ms)], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    total_ms = t.item()
    tokens = a.steps * cfg.global_batch_tokens
    gpu = r["trials"][0]["gpu"]
    if rank == 0:
        value = tokens / (total_ms / 1e3)
        print(json.dumps({
            "metric": "train tokens/s (device-timed, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": total_ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids in [0, 50257) in the reference shard format; random-init weights",
            "impl": "reference",
            "config": headline_config(micro, seq, world, par) if headline_config else {"global_batch": micro * dp, "seq_len": seq},
            "stack": "torch.compile default + mem_efficient SDPA + torch DDP/NCCL + foreach AdamW",
            "comparable": "e2e.value (both arms time their public train_step with the host copies inside the region)",
            # The reference's benchmark() times its real train_step: every step includes the pinned
            # H2D copy of the batch and the .item() reads of loss and grad norm, so its device-timed
            # number already is its end-to-end number.
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": micro * (seq + 1) * 8, "d2h_bytes_per_step": 8},
            "gpu_launches": 0,
            "clocks": {"sm_mhz": (gpu.get("sm_mhz") or {}).get("median"), "sm_max_mhz": None,
                       "reasons": gpu.get("slowdown_reasons", []), "n_samples": gpu.get("n_samples", 0)},
            "warmup_s": r["warmup_s"], "wall_s": wall, "loss_last": r["trials"][0]["loss_last"],
        }), flush=True)
    distributed.destroy()
    return 0
