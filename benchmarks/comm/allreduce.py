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
    world, rank = d.world, d.rank
    n_max = 114_150_144 // (256 * world * 8) * (256 * world * 8)
    buf = SymmetricBuffer(n_max, torch.float32, dev)
    ar = SymmetricAllReduce(buf)
    comm = ar.comm
    say = lambda *a: print(*a, flush=True) if rank == 0 else None
    # correctness once
    buf.tensor.copy_(torch.arange(n_max, device=dev, dtype=torch.float32) % 97 + rank)
    torch.cuda.synchronize(); dist.barrier()
    ar.all_reduce_(0, n_max, 1.0 / world)
    ar.check_status()
    want = torch.arange(n_max, device=dev, dtype=torch.float32) % 97 + (world - 1) / 2
    ok = torch.allclose(buf.tensor, want)
    plain = torch.zeros(n_max, device=dev)
    has_mc = bool(buf.multicast_ptr)
    say(f"# world {world}; roofline: measured peer copy 770 GB/s per direction per GPU; multicast address {'available' if has_mc else 'not available'}")
    say("## all-reduce, fp32 in place, fused 1/world scale + squared norm (bus GB/s = 2 (N-1)/N bytes / time)")
    say("size MiB | ours ms | bus GB/s | of 770 | ours multimem ms | bus GB/s | NCCL ms | bus GB/s")
    for mb in (4, 25, 100, 154, 435):
        n = min(n_max, mb * 2**20 // 4 // (world * 4) * (world * 4))
        bus = lambda t: 2 * (world - 1) / world * n * 4 / t / 1e6
        t_ours = timeit(lambda: comm.all_reduce_(buf, 0, n, 1.0 / world, False, 0))
        t_mc = timeit(lambda: comm.all_reduce_(buf, 0, n, 1.0 / world, True, 0)) if has_mc else float("nan")
        t_nccl = timeit(lambda: dist.all_reduce(plain[:n]))
        say(f"{n * 4 / 2**20:7.1f} | {t_ours:7.3f} | {bus(t_ours):6.1f} | {bus(t_ours) / 770:.2f} | {t_mc:7.3f} | {bus(t_mc):6.1f} | {t_nccl:7.3f} | {bus(t_nccl):6.1f}")
    comm.check_status()
    say("## reduce-scatter (fp32, + scale + squared norm) and all-gather (16-bit parameters) at the FSDP unit sizes (GB/s = (N-1)/N bytes / time)")
    say("collective | unit MiB | ours ms | GB/s | of 770 | NCCL ms | GB/s")
    for mb in (24, 147):   # a block unit (6.3 M parameters) and the root unit (38.6 M) in fp32
        n = min(n_max, mb * 2**20 // 4 // (world * 256) * (world * 256))
        per = n // world
        out, sq = torch.empty(per, device=dev), torch.zeros((), device=dev)
        gbs = lambda t, nbytes: (world - 1) / world * nbytes / t / 1e6
        t_ours = timeit(lambda: comm.reduce_scatter(buf, out, sq, 0, per, 1.0 / world, bucket=0))
        t_nccl = timeit(lambda: dist.reduce_scatter_tensor(out, plain[:n]))
        say(f"reduce-scatter | {n * 4 / 2**20:6.1f} | {t_ours:7.3f} | {gbs(t_ours, n * 4):6.1f} | {gbs(t_ours, n * 4) / 770:.2f} | {t_nccl:7.3f} | {gbs(t_nccl, n * 4):6.1f}")
        shards = SymmetricBuffer(per, torch.bfloat16, dev)
        full = torch.empty(n, device=dev, dtype=torch.bfloat16)
        t_ours = timeit(lambda: comm.all_gather(shards, full, 0, per * 2))
        t_nccl = timeit(lambda: dist.all_gather_into_tensor(full, shards.tensor))
        say(f"all-gather     | {n * 2 / 2**20:6.1f} | {t_ours:7.3f} | {gbs(t_ours, n * 2):6.1f} | {gbs(t_ours, n * 2) / 770:.2f} | {t_nccl:7.3f} | {gbs(t_nccl, n * 2):6.1f}")
        del shards
    comm.check_status()
    say("ALLREDUCE_OK" if ok else "ALLREDUCE_MISMATCH")
    parallel.destroy()


if __name__ == "__main__":
    main()
