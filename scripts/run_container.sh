#!/usr/bin/env bash
# Run a command inside the framework's container with every GPU visible and the repo mounted at /workspace.
#   scripts/run_container.sh python scripts/train.py --config configs/b200/single.yaml
# IMAGE defaults to the tag built by:  docker build -t nanonemo-b200 -f docker/Dockerfile .
# --ipc=host: NCCL and the pinned staging ring want shared memory; --ulimit memlock for pinned allocations.
set -euo pipefail
cd "$(dirname "$0")/.."
exec docker run --rm --gpus all --ipc=host --ulimit memlock=-1 --ulimit stack=67108864 \
  -e NANONEMO_CONTAINER="${IMAGE:-nanonemo-b200}" -e WANDB_MODE="${WANDB_MODE:-offline}" \
  -v "$PWD":/workspace -w /workspace "${IMAGE:-nanonemo-b200}" "$@"
