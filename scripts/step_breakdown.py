#!/usr/bin/env python
"""Where a training step spends its GPU time: kernel time per group from the PyTorch profiler (CUDA activity only).

    python scripts/step_breakdown.py --config configs/b200/single.yaml [--steps 3] [--set train.micro_batch=32]

Prints one row per kernel group (GEMMs, attention forward / backward, norms, SwiGLU, RoPE, cross-entropy, optimizer,
collectives, everything else) with milliseconds per step and the share of the total. Times come from the profiler's kernel
records, so they add up to busy GPU time, not to wall-clock step time.
"""

import argparse
import sys
from collections import defaultdict
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

GROUPS = [  # first match wins
    ("tcgen05 GEMM (CTA pair)", ("gemm2_tcgen05",)),
    ("tcgen05 GEMM (single CTA)", ("gemm_tcgen05",)),
    ("flash attention backward", ("flash_bwd", "flash_delta", "flash_dq_convert")),
    ("flash attention forward", ("flash_fwd",)),
    ("add + RMSNorm", ("rmsnorm", "dw_reduce")),
    ("SwiGLU", ("swiglu",)),
    ("RoPE", ("rope",)),
    ("cross-entropy", ("ce_inplace", "ce_stats", "ce_grad")),
    ("embedding", ("embedding",)),
    ("AdamW / grad norm", ("adamw", "sumsq")),
    ("collectives", ("allreduce", "reduce_scatter", "allgather", "all_gather", "nccl")),
    ("MXFP8 quantise", ("mxfp8",)),
    ("library GEMM", ("cutlass", "cublas", "nvjet", "gemm")),
]


def group_of(name: str) -> str:
    low = name.lower()
    for label, keys in GROUPS:
        if any(k in low for k in keys):
            return label
    return "other"


def main(argv=None):
    import torch
    from torch.profiler import ProfilerActivity, profile

    from nanonemo_b200 import parallel
    from nanonemo_b200.data.loader import DeviceBatches, TokenLoader
    from nanonemo_b200.train.config import apply_overrides, load_config
    from nanonemo_b200.train.optim import build_optimizer
    from nanonemo_b200.train.trainer import AMP_DTYPES, build_parallel, build_scaler, train_step

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--set", nargs="*", default=[], metavar="section.key=value")
    a = ap.parse_args(argv)
    model_cfg, cfg = apply_overrides(*load_config(a.config), a.set)
    d = parallel.init()
    if not d.device.startswith("cuda"):
        raise SystemExit("step_breakdown.py needs a CUDA device")
    strategy = build_parallel(model_cfg, cfg, d)
    opt = build_optimizer(strategy.model, cfg.peak_lr, cfg.weight_decay, store=strategy.store)
    amp, scaler = AMP_DTYPES[cfg.precision], build_scaler(cfg, d.device, strategy.sharded_grads)
    loader = TokenLoader(cfg.data_dir, "train", cfg.seq_len, cfg.micro_batch, seed=cfg.seed, rank=strategy.dp_rank,
                         world_size=strategy.dp_world, device=d.device)
    src, accum = DeviceBatches(loader, 4), cfg.grad_accum(strategy.dp_world)
    for _ in range(3):
        train_step(strategy, opt, src, accum, cfg.grad_clip, amp, scaler, host_sync=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            train_step(strategy, opt, src, accum, cfg.grad_clip, amp, scaler, host_sync=False)
        torch.cuda.synchronize()
    per_group, per_kernel = defaultdict(float), defaultdict(float)
    for ev in prof.key_averages():
        us = getattr(ev, "device_time_total", None) or getattr(ev, "cuda_time_total", 0.0)
        if us:
            per_group[group_of(ev.key)] += us / 1e3 / a.steps
            per_kernel[ev.key] += us / 1e3 / a.steps
    if d.main:
        total = sum(per_group.values())
        print(f"GPU kernel time per step: {total:.2f} ms over {a.steps} steps ({cfg.parallel}, world {d.world})")
        print("| group | ms / step | share |\n|---|---|---|")
        for label, ms in sorted(per_group.items(), key=lambda kv: -kv[1]):
            print(f"| {label} | {ms:.2f} | {100 * ms / total:.1f} % |")
        print("\ntop kernels:")
        for name, ms in sorted(per_kernel.items(), key=lambda kv: -kv[1])[:12]:
            print(f"  {ms:7.3f} ms  {name[:110]}")
    parallel.destroy()


if __name__ == "__main__":
    main()
