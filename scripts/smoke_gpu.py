#!/usr/bin/env python
"""GPU smoke test: environment, the kernel library, one tcgen05 GEMM against torch.matmul, and a tiny
training step on the sm100 path. Also usable as a small profiler target (a few hundred launches).

    python scripts/smoke_gpu.py
"""

import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from nanonemo_b200.utils.env import capture_env  # noqa: E402


def main():
    env = capture_env()
    print(json.dumps({k: env[k] for k in ("torch", "cuda_runtime", "nccl", "devices")}, indent=1))
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device")
    from nanonemo_b200.ops import _lib
    from nanonemo_b200.ops.gemm import check_status, gemm

    if not _lib.available():
        raise SystemExit(f"kernel library missing: build it with python -m nanonemo_b200.csrc.build ({_lib.LIB_PATH})")
    print("kernel library:", _lib.LIB_PATH, "arch", _lib.lib().nnb_build_arch())
    a = torch.randn(1024, 768, device="cuda").bfloat16()
    b = torch.randn(1280, 768, device="cuda").bfloat16()
    out = gemm(a, b)
    check_status()
    ref = a.float() @ b.float().t()
    err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
    print(f"tcgen05 GEMM 1024x1280x768: max relative error {err:.2e} (tensor-core path: tcgen05.mma + TMA + TMEM)")
    assert err < 2e-2
    import __graft_entry__ as entry

    entry.smoke()


if __name__ == "__main__":
    main()
