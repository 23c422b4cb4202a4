"""Single-kernel GEMM -> reduce-scatter and all-gather -> GEMM on two real GPUs (peer memory over NVLink)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = Path(__file__).resolve().parent


def test_fused_collective_gemms_match_nccl_plus_matmul():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29571", str(HERE / "fused_gemm_worker.py")], env=env, capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "FUSED_GEMM_OK" in r.stdout, r.stdout[-3000:]
