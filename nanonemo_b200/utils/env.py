"""Software / hardware environment recorded with every result (cf. nanonemo/utils/env.py:1-95)."""

import datetime
import json
import os
import platform
import socket
import subprocess
from pathlib import Path

_SMI_QUERY = ("name", "driver_version", "clocks.sm", "clocks.mem", "clocks.max.sm", "temperature.gpu",
              "power.draw", "power.limit", "clocks_event_reasons.active")


def _run(cmd: list[str], timeout: float = 20.0) -> str | None:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, check=True, timeout=timeout).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        return None


def gpu_slug() -> str:
    """Short GPU name for result folders: "b200", "t4", "cpu"."""
    import torch

    if not torch.cuda.is_available():
        return "cpu"
    words = torch.cuda.get_device_name().lower().replace("laptop gpu", "").split()
    return "-".join(w for w in words if w not in ("nvidia", "geforce", "tesla"))


def git_info() -> dict:
    root = str(Path(__file__).resolve().parents[2])
    commit = _run(["git", "-C", root, "rev-parse", "HEAD"])
    status = _run(["git", "-C", root, "status", "--porcelain"])
    return {"commit": commit, "dirty": None if status is None else bool(status)}


def gpu_state() -> list[dict]:
    out = _run(["nvidia-smi", f"--query-gpu={','.join(_SMI_QUERY)}", "--format=csv,noheader,nounits"])
    if not out:
        return []
    return [dict(zip(_SMI_QUERY, (c.strip() for c in row.split(",")))) for row in out.splitlines()]


def measured_peaks() -> dict | None:
    """Peaks measured on this pool's GPUs (MEASURED_PEAKS.json at the repository root), if present."""
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return json.loads(path.read_text())
    except (OSError, ValueError):
        return None


def capture_env() -> dict:
    import torch

    try:
        import triton

        triton_version = triton.__version__
    except ImportError:
        triton_version = None
    cuda = torch.cuda.is_available()
    devices = []
    for i in range(torch.cuda.device_count() if cuda else 0):
        p = torch.cuda.get_device_properties(i)
        devices.append({"name": p.name, "capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                        "memory_gb": round(p.total_memory / 2**30, 2), "l2_mb": round(p.L2_cache_size / 2**20, 1)})
    return {
        "timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat(),
        "host": socket.gethostname(),
        "python": platform.python_version(),
        "torch": torch.__version__,
        "triton": triton_version,
        "cuda_runtime": torch.version.cuda,
        "cudnn": torch.backends.cudnn.version() if cuda else None,
        "nccl": ".".join(map(str, torch.cuda.nccl.version())) if cuda else None,
        "container": os.environ.get("NVIDIA_PYTORCH_VERSION"),
        "devices": devices,
        "gpu_state": gpu_state(),
        "git": git_info(),
    }


if __name__ == "__main__":
    print(json.dumps(capture_env(), indent=2))
