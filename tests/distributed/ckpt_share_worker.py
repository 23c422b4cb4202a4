"""Worker of test_parallel.py::test_each_rank_saves_its_share_only: under every layout the state a rank hands to the checkpoint
writer is about 1 / world of the full state (its row block of every tensor), never a gathered copy of the whole."""

import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from nanonemo_b200 import parallel  # noqa: E402
from nanonemo_b200.models.config import ModelConfig  # noqa: E402
from nanonemo_b200.train.checkpoint import collect_state  # noqa: E402
from nanonemo_b200.train.config import TrainConfig  # noqa: E402
from nanonemo_b200.train.optim import build_optimizer  # noqa: E402
from nanonemo_b200.train.trainer import build_parallel  # noqa: E402


def local_numel(tree) -> int:
    if isinstance(tree, dict):
        return sum(local_numel(v) for v in tree.values())
    if hasattr(tree, "to_local"):
        return tree.to_local().numel()
    return tree.numel() if torch.is_tensor(tree) else 0


def main():
    d = parallel.init()
    mc = ModelConfig(n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, d_ff=384, vocab_size=50304, max_seq_len=128)
    for par in ("ddp", "fsdp", "tp"):
        cfg = TrainConfig(data_dir="synthetic", out_dir="runs/share", seq_len=128, micro_batch=2, global_batch_tokens=1024, parallel=par)
        torch.manual_seed(0)
        strategy = build_parallel(mc, cfg, d)
        opt = build_optimizer(strategy.model, 1e-3, 0.1, store=strategy.store)
        state = collect_state(strategy, opt)
        full = sum(int(torch.Size(shape).numel()) for _, shape in strategy.checkpoint_names())
        # weights (+ the tied head's second name) and the two moments
        tied = mc.vocab_size * mc.d_model
        want = (3 * full + tied) / d.world
        got = local_numel(state["model"]) + local_numel(state["optim"]["state"])
        ok = want * 0.98 <= got <= want * 1.02 + 4 * len(state["model"]) * d.world
        if d.main:
            print(f"SHARE {par}: local {got} of {3 * full + tied} = {got / (3 * full + tied):.3f} ({'ok' if ok else 'TOO MUCH'})", flush=True)
        flag = torch.tensor([0.0 if ok else 1.0])
        dist.all_reduce(flag)
        if flag.item():
            sys.exit(1)
    if d.main:
        print("SHARE_OK", flush=True)
    parallel.destroy()


if __name__ == "__main__":
    main()
