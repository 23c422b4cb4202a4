#!/usr/bin/env bash
# Nsight Compute capture of one kernel family on a small case, and a text summary of the counters that
# matter (DRAM bytes / throughput, tensor-pipe activity, registers, achieved warps).
#   benchmarks/kernels/ncu.sh gemm 'regex:gemm_tcgen05' out_dir [tag]
# The target runs once without the profiler first; the capture is 3 launches of one kernel and never
# changes GPU clocks (--clock-control none). Several small targets can share one process and one capture:
#   NCU_COUNT=24 NCU_ITERS=2 benchmarks/kernels/ncu.sh rope,embedding,quantize 'regex:rope_packed|embedding_|quantize' out_dir small
# (NCU_COUNT launches matching the pattern, after NCU_SKIP of them; NCU_ITERS calls of each target).
set -euo pipefail
target=${1:?target: gemm|gemm_single|gemm_mxfp8|gemm_swiglu|gemm_swiglu_bwd|gemm_rope|flash|flash128|rmsnorm|swiglu|rope|ce|adamw|embedding|quantize}
pattern=${2:?kernel name pattern, e.g. regex:gemm_tcgen05}
out=${3:-ncu_out}
tag=${4:-$target}   # name of the output files (several kernels of one target can be captured one after the other)
here=$(cd "$(dirname "$0")" && pwd)
mkdir -p "$out"
iters=${NCU_ITERS:-4}
python "$here/ncu_target.py" "$target" "$iters" > "$out/${tag}_plain.log" 2>&1 &&
ncu --set full --clock-control none -k "$pattern" -s "${NCU_SKIP:-1}" -c "${NCU_COUNT:-3}" -o "$out/${tag}" -f python "$here/ncu_target.py" "$target" "$iters" > "$out/${tag}_ncu.log" 2>&1
ncu -i "$out/${tag}.ncu-rep" --page raw --csv > "$out/${tag}_raw.csv"
python "$here/ncu_table.py" "$out/${tag}_raw.csv" > "$out/${tag}_summary.txt"
cat "$out/${tag}_summary.txt"
