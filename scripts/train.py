#!/usr/bin/env python
"""Train from a YAML config.

    python scripts/train.py --config configs/smoke.yaml
    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=8 \
        scripts/train.py --config configs/dist/ddp.yaml [--set train.max_steps=20 model.attn_kernel=sm100]
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from nanonemo_b200 import parallel  # noqa: E402
from nanonemo_b200.train.config import apply_overrides, load_config  # noqa: E402
from nanonemo_b200.train.trainer import train  # noqa: E402


def console(record: dict) -> None:
    if record.get("event") == "start":
        print(f"start: {record['params']:,} params, {record['total_steps']} steps, accum {record['grad_accum']}, "
              f"{record['parallel']} x{record['world']} on {record['device']}"
              + (f", resumed from {record['resumed_from']}" if record.get("resumed_from") else ""), flush=True)
    elif "val_loss" in record:
        print(f"step {record['step']:>6}  val_loss {record['val_loss']:.4f}", flush=True)
    elif "event" in record:
        print(f"step {record['step']:>6}  [{record['event']}] {record.get('reason', '')}", flush=True)
    else:
        extra = f"  mfu {100 * record['mfu']:.1f}%" if "mfu" in record else ""
        print(f"step {record['step']:>6}  loss {record['loss']:.4f}  lr {record['lr']:.2e}  "
              f"gnorm {record['grad_norm']:.3f}  {record['tokens_per_s']:,.0f} tok/s{extra}", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--set", nargs="*", default=[], metavar="section.key=value",
                    help="override config values, e.g. train.max_steps=10 model.norm_kernel=sm100")
    a = ap.parse_args(argv)
    model_cfg, cfg = apply_overrides(*load_config(a.config), a.set)

    sinks = [console]
    if cfg.wandb_project:
        import os

        if int(os.environ.get("RANK", "0")) == 0:
            from nanonemo_b200.train.wandb_sink import WandbSink

            sinks.append(WandbSink(cfg.wandb_project, cfg.wandb_run_name, model_cfg, cfg))

    def log_fn(record):
        for s in sinks:
            s(record)

    try:
        train(model_cfg, cfg, log_fn=log_fn)
    finally:
        for s in sinks:
            if hasattr(s, "close"):
                s.close()
        parallel.destroy()


if __name__ == "__main__":
    main()
