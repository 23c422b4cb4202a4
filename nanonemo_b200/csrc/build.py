"""Ahead-of-time build of the kernel library: every ``*.cu`` in this folder -> one shared library.

    python -m nanonemo_b200.csrc.build [--force] [--verbose]

Each translation unit is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo``
(nvcc cross-compiles without a GPU) and the objects are linked into ``libnanonemo_b200.so`` next to
the sources, where ``nanonemo_b200.ops._lib`` loads it. Only the CUDA runtime and the driver API
(resolved at run time through cudaGetDriverEntryPoint) are needed: no torch headers, so a full
rebuild takes seconds. Objects are rebuilt when their source or a header is newer.
"""

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libnanonemo_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-DNNB_ARCH=100",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]
# Translation units whose arithmetic has to match a PyTorch reference operation for operation (the optimizer update):
# IEEE division and square root, no flush-to-zero. They are bandwidth-bound, so this costs nothing measurable.
PRECISE = {"adamw.cu", "comm.cu"}  # comm.cu: the reduce-scatter that applies AdamW in its epilogue


def nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _stale(obj: Path, deps: list[Path]) -> bool:
    return not obj.exists() or any(d.stat().st_mtime > obj.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h")) + sorted(HERE.glob("*.inc"))
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    jobs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        extra = os.environ.get("NANONEMO_NVCC_EXTRA", "").split()  # e.g. -DNNB_PROFILE: in-kernel phase timers of the attention kernels
        flags = [f for f in NVCC_FLAGS if not (src.name in PRECISE and f == "--use_fast_math")]
        cmd = [nvcc(), *ARCH_FLAGS, *flags, *extra, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (objdir / (src.stem + ".ptxas.log")).write_text(r.stderr)
        return src, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, r in pool.map(compile_one, jobs):
            if r.returncode != 0:
                failed = True
                print(f"--- {src.name} FAILED\n{r.stdout}\n{r.stderr}", file=sys.stderr)
            elif verbose:
                print(f"--- {src.name}\n{r.stderr}")
    if failed:
        raise RuntimeError("nvcc failed")
    objs = [objdir / (s.stem + ".o") for s in sources()]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    print(build(a.force, a.verbose))


if __name__ == "__main__":
    main()
