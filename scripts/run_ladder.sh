#!/usr/bin/env bash
# Benchmark the optimisation ladder, one process per stage, then print the table.
#   scripts/run_ladder.sh [stage-name ...]      env: DATA_DIR (default: synthetic), STEPS, TRIALS, EXTRA (extra --set overrides)
# A stage whose result carries throttle flags is re-run up to ATTEMPTS times after resting REST_S seconds
# (clock drops on a shared or power-capped GPU make stages incomparable). GPU clocks are only read, never set.
set -euo pipefail
cd "$(dirname "$0")/.."
stages=("$@")
[ ${#stages[@]} -eq 0 ] && stages=($(ls configs/stages | sed 's/\.yaml$//'))
for s in "${stages[@]}"; do
  for attempt in $(seq 1 "${ATTEMPTS:-2}"); do
    python scripts/bench_train.py --config "configs/stages/$s.yaml" --data-dir "${DATA_DIR:-synthetic}" \
      --steps "${STEPS:-50}" --trials "${TRIALS:-3}" ${EXTRA:+--set $EXTRA} | tee /tmp/ladder_$s.log
    grep -q "flags:" /tmp/ladder_$s.log || break
    echo "stage $s flagged; resting ${REST_S:-60}s before attempt $((attempt + 1))"; sleep "${REST_S:-60}"
  done
done
python scripts/ladder_table.py
