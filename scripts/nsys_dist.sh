#!/usr/bin/env bash
# Timeline of one multi-GPU benchmark config with Nsight Systems, and the share of GPU kernel time that went to
# communication kernels (NCCL's and this framework's own all-reduce / reduce-scatter / all-gather / fused-GEMM kernels).
#
#   scripts/nsys_dist.sh configs/b200/ddp.yaml [nproc] [extra scripts/bench_train.py arguments]
#
# What it does: runs scripts/bench_train.py under `nsys profile` with the capture range tied to cudaProfilerStart/Stop
# (NANONEMO_PROFILE=1 makes the benchmark open that window around its first timed trial only, so warm-up and compilation stay
# out of the trace), exports the per-kernel summary as CSV and hands it to scripts/comm_share.py. Outputs go to
# results/nsys/<gpu>-x<nproc>/<config>.{nsys-rep,bench.json} and <config>_cuda_gpu_kern_sum.csv.
#
# Reading the result: the share says how much kernel time was communication, not how much of it was exposed; for that
# compare the step time with the 1-GPU run at the same per-GPU work (bench.py prints both), or open the .nsys-rep and look
# at the side stream against the compute stream. Never wrap a number you want to quote in nsys: profile runs are for shares.
#
# Needs `nsys` on the PATH. Where it is not installed the script says so and exits 3; the launch list of
# `ncu --metrics gpu__time_duration.sum --clock-control none --csv` is an accepted input of scripts/comm_share.py as well.
set -euo pipefail
cd "$(dirname "$0")/.."

cfg=${1:?usage: scripts/nsys_dist.sh <config.yaml> [nproc] [bench_train.py arguments]}
nproc=${2:-2}
shift $(( $# < 2 ? $# : 2 ))

if ! command -v nsys >/dev/null 2>&1; then
    echo "nsys is not installed on this machine: no timeline taken." >&2
    echo "Kernel-time shares without nsys: python scripts/step_breakdown.py --config $cfg   (PyTorch profiler, one rank)" >&2
    exit 3
fi

name=$(basename "$cfg" .yaml)
gpu=$(python -c "from nanonemo_b200.utils.env import gpu_slug; print(gpu_slug())")
out="results/nsys/${gpu}-x${nproc}"
mkdir -p "$out"

NANONEMO_PROFILE=1 NANONEMO_NVTX=1 nsys profile --trace=cuda,nvtx,osrt --capture-range=cudaProfilerApi --capture-range-end=stop \
    --force-overwrite=true --output="$out/$name" \
    python -m torch.distributed.run --nnodes=1 --nproc-per-node="$nproc" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29511}" \
    scripts/bench_train.py --config "$cfg" --steps 5 --trials 1 --out "$out/$name.bench.json" "$@"

nsys stats --report cuda_gpu_kern_sum --format csv --output "$out/$name" --force-export=true "$out/$name.nsys-rep" >/dev/null
python scripts/comm_share.py "$out/${name}_cuda_gpu_kern_sum.csv"
