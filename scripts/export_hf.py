#!/usr/bin/env python
"""Export a training checkpoint to Hugging Face Llama format.

    python scripts/export_hf.py --ckpt runs/main/ckpt --out export/nanonemo-114m [--config runs/main/config.yaml] [--no-tokenizer]
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from nanonemo_b200.eval.hf_export import export, load_checkpoint  # noqa: E402
from nanonemo_b200.train.checkpoint import find_latest  # noqa: E402
from nanonemo_b200.train.config import load_config  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ckpt", required=True, help="a checkpoint directory, or a root holding a `latest` file")
    ap.add_argument("--out", required=True)
    ap.add_argument("--config", default=None, help="default: config.yaml of the run the checkpoint belongs to")
    ap.add_argument("--no-tokenizer", action="store_true", help="skip saving the GPT-2 tokenizer (needs a cached copy)")
    a = ap.parse_args(argv)
    path = find_latest(a.ckpt)
    if path is None:
        raise SystemExit(f"no complete checkpoint under {a.ckpt}")
    config = Path(a.config) if a.config else next((p / "config.yaml" for p in path.parents if (p / "config.yaml").exists()), None)
    if config is None:
        raise SystemExit("cannot find the run's config.yaml; pass --config")
    model_cfg, _ = load_config(config)
    out = export(load_checkpoint(path, model_cfg), a.out, tokenizer=not a.no_tokenizer)
    print(f"exported {path} -> {out}")


if __name__ == "__main__":
    main()
