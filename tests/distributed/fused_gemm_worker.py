"""Worker of test_fused_gemm_multigpu.py: one process per GPU; checks the single-kernel GEMM->reduce-scatter
and all-gather->GEMM against torch.distributed collectives + matmul and prints timings."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from nanonemo_b200 import parallel  # noqa: E402
from nanonemo_b200.ops.gemm import FusedCollectiveGemm, gemm  # noqa: E402
from nanonemo_b200.parallel.symm import SymmetricBuffer  # noqa: E402


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
    rank, world = d.rank, d.world
    dev = torch.device(d.device)
    torch.manual_seed(1234)  # same on every rank
    M = int(os.environ.get("FG_M", "16384"))
    fused = FusedCollectiveGemm(dev, dist.group.WORLD, rank, world)
    ok = True
    # ---------------- GEMM -> reduce-scatter (row parallel: K is sharded)
    for (N, K) in ((768, 768), (768, 2048)):
        a_full = torch.randn(M, K, device=dev).bfloat16()
        b_full = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        kl = K // world
        a_loc, b_loc = a_full[:, rank * kl:(rank + 1) * kl].contiguous(), b_full[:, rank * kl:(rank + 1) * kl].contiguous()
        out = SymmetricBuffer((M // world) * N, torch.bfloat16, dev)
        got = fused.gemm_rs(a_loc, b_loc, out).clone()
        fused.check_status()
        ref = (a_full.float() @ b_full.float().t())[rank * (M // world):(rank + 1) * (M // world)]
        err = (got.float() - ref).abs().max().item() / ref.abs().max().item()
        ok &= err < 3e-2

        def baseline():
            part = gemm(a_loc, b_loc)
            o = torch.empty(M // world, N, dtype=torch.bfloat16, device=dev)
            dist.reduce_scatter_tensor(o, part)
            return o

        t_f, t_b = timeit(lambda: fused.gemm_rs(a_loc, b_loc, out)), timeit(baseline)
        if rank == 0:
            print(f"gemm_rs M={M} N={N} K={K}/{world}: rel err {err:.2e}; fused {t_f:.3f} ms vs gemm + NCCL reduce-scatter {t_b:.3f} ms", flush=True)
    # ---------------- all-gather -> GEMM (column parallel: N is sharded, A rows arrive from peers)
    for (N, K) in ((1280, 768), (4096, 768)):
        nl = N // world
        a_full = torch.randn(M, K, device=dev).bfloat16()
        b_loc = (torch.randn(nl, K, device=dev) * 0.05).bfloat16()
        buf = SymmetricBuffer(M * K, torch.bfloat16, dev)
        rows = M // world
        mine = buf.tensor.view(M, K)
        mine.zero_()
        mine[rank * rows:(rank + 1) * rows].copy_(a_full[rank * rows:(rank + 1) * rows])
        torch.cuda.synchronize()
        dist.barrier()
        got = fused.ag_gemm(buf, M, K, b_loc).clone()
        fused.check_status()
        ref = a_full.float() @ b_loc.float().t()
        err = (got.float() - ref).abs().max().item() / ref.abs().max().item()
        ok &= err < 3e-2
        shard = a_full[rank * rows:(rank + 1) * rows].contiguous()

        def baseline():
            full = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
            dist.all_gather_into_tensor(full, shard)
            return gemm(full, b_loc)

        t_f, t_b = timeit(lambda: fused.ag_gemm(buf, M, K, b_loc)), timeit(baseline)
        if rank == 0:
            print(f"ag_gemm M={M} N={N}/{world} K={K}: rel err {err:.2e}; fused {t_f:.3f} ms vs NCCL all-gather + gemm {t_b:.3f} ms", flush=True)
    flag = torch.tensor([float(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("FUSED_GEMM_OK" if flag.item() == 1.0 else "FUSED_GEMM_MISMATCH", flush=True)
    parallel.destroy()


if __name__ == "__main__":
    main()
