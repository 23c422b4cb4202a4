"""In-place fp32 all-reduce (+ 1/world scale) over symmetric memory: this framework's two-shot kernel vs NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29590 benchmarks/comm/allreduce.py

Timing: CUDA events on the launching stream, 3 warm-up + 10 timed calls, MAX over ranks. Bus bandwidth =
2 (N-1)/N x bytes / time (the NCCL convention); the roofline is the measured 770 GB/s per direction.
"""

import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from nanonemo_b200 import parallel  # noqa: E402
from nanonemo_b200.parallel.symm import SymmetricAllReduce, SymmetricBuffer  # noqa: E402


def timeit(fn, iters=10):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    d = parallel.init()
    dev = torch.device(d.device)
    world = d.world
    n_max = 114_150_144 // (256 * world * 8) * (256 * world * 8)
    buf = SymmetricBuffer(n_max, torch.float32, dev)
    ar = SymmetricAllReduce(buf)
    # correctness once
    buf.tensor.copy_(torch.arange(n_max, device=dev, dtype=torch.float32) % 97 + d.rank)
    torch.cuda.synchronize(); dist.barrier()
    ar.all_reduce_(0, n_max, 1.0 / world)
    ar.check_status()
    want = torch.arange(n_max, device=dev, dtype=torch.float32) % 97 + (world - 1) / 2
    ok = torch.allclose(buf.tensor, want)
    plain = torch.zeros(n_max, device=dev)
    for mb in (4, 25, 100, 154, 435):
        n = min(n_max, mb * 2**20 // 4 // (world * 4) * (world * 4))
        t_ours = timeit(lambda: ar.all_reduce_(0, n, 1.0 / world))
        t_nccl = timeit(lambda: dist.all_reduce(plain[:n]))
        bus = lambda t: 2 * (world - 1) / world * n * 4 / t / 1e6
        if d.rank == 0:
            print(f"{n * 4 / 2**20:7.1f} MiB  ours {t_ours:7.3f} ms ({bus(t_ours):6.1f} GB/s bus, {bus(t_ours) / 770:.2f} of 770)   "
                  f"NCCL {t_nccl:7.3f} ms ({bus(t_nccl):6.1f} GB/s bus)", flush=True)
    if d.rank == 0:
        print("ALLREDUCE_OK" if ok else "ALLREDUCE_MISMATCH", flush=True)
    parallel.destroy()


if __name__ == "__main__":
    main()
