#!/usr/bin/env python
"""Zero-shot evaluation of an exported model with lm-evaluation-harness (needs the `lm_eval` package
and its datasets; neither is available offline).

    python scripts/eval.py --model export/nanonemo-114m --name nanonemo [--tasks hellaswag arc_easy piqa lambada_openai]
"""

import argparse
import json
from pathlib import Path

TASKS = ["hellaswag", "arc_easy", "piqa", "lambada_openai"]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="HF model directory or hub id (e.g. gpt2)")
    ap.add_argument("--name", required=True)
    ap.add_argument("--tasks", nargs="*", default=TASKS)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--out-dir", default="results/eval")
    a = ap.parse_args(argv)
    try:
        import lm_eval
    except ImportError as e:
        raise SystemExit("lm_eval is not installed: pip install lm-eval==0.4.9 (needs network)") from e
    res = lm_eval.simple_evaluate(model="hf", model_args=f"pretrained={a.model},dtype=float32", tasks=a.tasks,
                                  num_fewshot=0, batch_size=a.batch_size, limit=a.limit)
    summary = {"model": a.model, "tasks": {t: {k: v for k, v in m.items() if isinstance(v, (int, float))}
                                           for t, m in res["results"].items()}}
    out = Path(a.out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / f"{a.name}.json").write_text(json.dumps(summary, indent=1))
    print(json.dumps(summary["tasks"], indent=1))


if __name__ == "__main__":
    main()
