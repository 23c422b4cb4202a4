#!/usr/bin/env bash
# Nsight Compute capture of one kernel family on a small case, and a text summary of the counters that
# matter (DRAM bytes / throughput, tensor-pipe activity, registers, achieved warps).
#   benchmarks/kernels/ncu.sh gemm 'regex:gemm_tcgen05' out_dir
# The target runs once without the profiler first; the capture is 3 launches of one kernel and never
# changes GPU clocks (--clock-control none).
set -euo pipefail
target=${1:?target: gemm|gemm_single|gemm_mxfp8|flash|flash128|rmsnorm|swiglu|rope|ce|adamw}
pattern=${2:?kernel name pattern, e.g. regex:gemm_tcgen05}
out=${3:-ncu_out}
here=$(cd "$(dirname "$0")" && pwd)
mkdir -p "$out"
python "$here/ncu_target.py" "$target" 4 > "$out/${target}_plain.log" 2>&1 &&
ncu --set full --clock-control none -k "$pattern" -s 1 -c 3 -o "$out/${target}" -f python "$here/ncu_target.py" "$target" 4 > "$out/${target}_ncu.log" 2>&1
ncu -i "$out/${target}.ncu-rep" --page raw --csv > "$out/${target}_raw.csv"
python "$here/ncu_table.py" "$out/${target}_raw.csv" > "$out/${target}_summary.txt"
cat "$out/${target}_summary.txt"
