#!/usr/bin/env bash
# Benchmark the precision configs (fp16 / bf16 / bf16 on the GEMM kernels / fp8 recipes) one process each, then print the table.
#   scripts/run_precision.sh        env: DATA_DIR (default: synthetic), STEPS, TRIALS
# fp8 runs the MXFP8 block linears (precision: fp8 needs linear_impl: mxfp8 or te; both resolve to the same kernels here).
set -euo pipefail
cd "$(dirname "$0")/.."
for f in configs/precision/*.yaml; do
  python scripts/bench_train.py --config "$f" --data-dir "${DATA_DIR:-synthetic}" --steps "${STEPS:-50}" --trials "${TRIALS:-3}" \
    --out "results/precision/$(basename "$f" .yaml).json"
done
python scripts/ladder_table.py results/precision
