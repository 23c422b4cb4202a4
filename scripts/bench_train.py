#!/usr/bin/env python
"""Benchmark the training step of a YAML config; writes results/<ladder|dist>/<gpu>[-xN]/<config>.json.

    python scripts/bench_train.py --config configs/stages/s3_compile.yaml --steps 50 --trials 3
    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=8 \
        scripts/bench_train.py --config configs/dist/ddp.yaml
"""

import argparse
import json
import sys
from dataclasses import replace
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from nanonemo_b200 import parallel  # noqa: E402
from nanonemo_b200.train.bench import benchmark  # noqa: E402
from nanonemo_b200.train.config import apply_overrides, load_config  # noqa: E402
from nanonemo_b200.utils.env import gpu_slug  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--trials", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--out", default=None, help="output JSON path (default: under results/)")
    ap.add_argument("--data-dir", default=None, help="override train.data_dir ('synthetic' needs no files)")
    ap.add_argument("--set", nargs="*", default=[], metavar="section.key=value")
    a = ap.parse_args(argv)
    model_cfg, cfg = apply_overrides(*load_config(a.config), a.set)
    if a.data_dir:
        cfg = replace(cfg, data_dir=a.data_dir)
    try:
        result = benchmark(model_cfg, cfg, steps=a.steps, trials=a.trials, warmup_steps=a.warmup)
        d = parallel.init()
        if d.main:
            if a.out:
                out = Path(a.out)
            else:
                kind = "ladder" if cfg.parallel == "none" and "stages" in a.config else "dist"
                folder = gpu_slug() + (f"-x{d.world}" if kind == "dist" else "")
                out = Path("results") / kind / folder / (Path(a.config).stem + ".json")
            out.parent.mkdir(parents=True, exist_ok=True)
            out.write_text(json.dumps(result, indent=1))
            t, m = result["tokens_per_s"], result["mfu"]
            print(f"{Path(a.config).stem}: {t['median']:,.0f} tok/s (min {t['min']:,.0f}, max {t['max']:,.0f}), "
                  f"step {result['step_ms']['median']:.2f} ms"
                  + (f", MFU {100 * next(iter(m.values()))['median']:.1f}%" if m else "")
                  + (f", flags: {result['throttle_flags']}" if result["throttle_flags"] else ""))
            print(f"wrote {out}")
    finally:
        parallel.destroy()


if __name__ == "__main__":
    main()
