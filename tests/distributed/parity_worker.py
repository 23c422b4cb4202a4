"""Worker of test_multigpu.py::test_layouts_and_collectives_at_world_size: one process per GPU under torch.distributed.run.

Part 1 checks the collective kernels (csrc/comm.cu) for this world size against exact expected values: every rank fills its
buffer with small integers, so fp32 sums are exact whatever the order, and the all-reduce / reduce-scatter / all-gather results
and the in-kernel squared norm must match to the last bit. Part 2 trains a small model for a few optimizer steps under every
layout this world size admits (ddp, ddp replayed from a CUDA graph, fsdp, tp with rank pairs when the KV heads do not divide,
the 2-D fsdp x tp mesh) on the SAME global batch and compares the per-step losses with a single-GPU run done in the same
process. Prints one line per check and PARITY_OK at the end (rank 0)."""

import gc
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from nanonemo_b200 import parallel  # noqa: E402
from nanonemo_b200.data.loader import TokenLoader  # noqa: E402
from nanonemo_b200.models.config import ModelConfig  # noqa: E402
from nanonemo_b200.parallel.symm import SymmetricAllReduce, SymmetricBuffer, SymmetricComm  # noqa: E402
from nanonemo_b200.train.config import TrainConfig  # noqa: E402
from nanonemo_b200.train.optim import build_optimizer  # noqa: E402
from nanonemo_b200.train.trainer import AMP_DTYPES, build_parallel, train_step  # noqa: E402

STEPS, SEQ, GLOBAL_SEQS, MICRO = 4, 256, 32, 4
MODEL = dict(n_layers=2, d_model=512, n_heads=8, n_kv_heads=4, d_ff=1024, vocab_size=50304, max_seq_len=SEQ)
TOL = 2e-2


def say(*a):
    if dist.get_rank() == 0:
        print(*a, flush=True)


def check_collectives(d):
    rank, world, dev = d.rank, d.world, torch.device(d.device)
    ok = True
    for n in (4096, (1 << 20) + 4 * world * 13, 3_000_000 // (4 * world) * (4 * world)):
        n -= n % (4 * world)
        buf = SymmetricBuffer(n, torch.float32, dev)
        ar = SymmetricAllReduce(buf)
        base = (torch.arange(n, device=dev) % 7).float()
        expect = base * world + sum(range(world))  # rank r holds base + r
        for rep in range(2):  # twice: the device-resident epochs must carry over
            buf.tensor.copy_(base + rank)
            torch.cuda.synchronize()
            dist.barrier()
            ar.all_reduce_(0, n, 1.0, bucket=rep)
            got_norm = ar.norm_sq(rep + 1)
            ar.check_status()
            same = torch.equal(buf.tensor, expect)
            want_norm = expect.double().pow(2).sum().item() * (rep + 1)
            ok &= same and abs(got_norm.item() - want_norm) <= 1e-5 * want_norm
            say(f"  all_reduce n={n} rep={rep}: exact={same} norm {got_norm.item():.6e} vs {want_norm:.6e}")
        # reduce-scatter + all-gather on the same communicator
        comm = ar.comm
        per = n // world
        buf.tensor.copy_(base + rank)
        out = torch.empty(per, device=dev)
        sumsq = torch.zeros((), device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        comm.reduce_scatter(buf, out, sumsq, 0, per, 0.5)
        want = expect[rank * per:(rank + 1) * per] * 0.5
        rs_ok = torch.equal(out, want) and abs(sumsq.item() - want.double().pow(2).sum().item()) <= 1e-5 * sumsq.item()
        shards = SymmetricBuffer(per, torch.float32, dev)
        shards.tensor.copy_(base[:per] * (rank + 1))
        full = torch.empty(n, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        comm.all_gather(shards, full, 0, per * 4)
        comm.check_status()
        ag_ok = all(torch.equal(full[r * per:(r + 1) * per], base[:per] * (r + 1)) for r in range(world))
        ok &= rs_ok and ag_ok
        say(f"  reduce_scatter n={n}: exact={rs_ok}   all_gather: exact={ag_ok}")
        del ar, comm, buf, shards
    return ok and check_vocab_parallel_embedding(d)


def check_vocab_parallel_embedding(d):
    """Forward rows and table gradient of the vocabulary-parallel embedding kernels against index arithmetic on the full table
    (integer-valued data: the scatter-add is exact in any order). Run twice per dtype: the staging buffer is reused."""
    rank, world, dev = d.rank, d.world, torch.device(d.device)
    V, D, per = 64, 72, 300  # rows per rank, width (multiple of 8), tokens per rank (not a multiple of the block count)
    comm = SymmetricComm(dev, None, rank, world)
    stage = SymmetricBuffer(per * D, torch.float32, dev)
    gen = torch.Generator().manual_seed(5)
    table = torch.randint(-8, 9, (V * world, D), generator=gen).float().to(dev)
    ok = True
    for dtype in (torch.float32, torch.bfloat16):
        for rep in range(2):
            idx = torch.randint(0, V * world, (per * world,), generator=gen).to(dev)
            grads = torch.randint(-4, 5, (per * world, D), generator=gen).to(dev).to(dtype)
            out = torch.empty((per, D), dtype=dtype, device=dev)
            torch.cuda.synchronize()
            dist.barrier()
            comm.vp_embedding(stage, idx, out, table[rank * V:(rank + 1) * V].contiguous(), rank * V, backward=False)
            dW = torch.ones((V, D), device=dev)
            comm.vp_embedding(stage, idx, grads[rank * per:(rank + 1) * per].contiguous(), dW, rank * V, backward=True)
            comm.check_status()
            want = table[idx[rank * per:(rank + 1) * per]].to(dtype)
            want_dW = torch.ones((V * world, D), device=dev).index_add_(0, idx, grads.float())[rank * V:(rank + 1) * V]
            good = torch.equal(out, want) and torch.equal(dW, want_dW)
            ok &= good
            say(f"  vocab-parallel embedding {str(dtype)[6:]} rep={rep}: exact={good}")
    return ok


def run_layout(d, par, extra=None, fake_single=False):
    """-> per-step losses of STEPS optimizer steps on the fixed global batch."""
    cfgs = dict(data_dir="synthetic", out_dir="runs/parity", seq_len=SEQ, micro_batch=MICRO, global_batch_tokens=GLOBAL_SEQS * SEQ,
                total_tokens=10**9, peak_lr=1e-3, precision="bf16", parallel=par, eval_every=10**9, fsdp_prefetch=True, comm="fused")
    cfgs.update(extra or {})
    cfg = TrainConfig(**cfgs)
    who = parallel.Dist(device=d.device) if fake_single else d
    torch.manual_seed(0)
    strategy = build_parallel(ModelConfig.sm100(**MODEL), cfg, who)
    opt = build_optimizer(strategy.model, cfg.peak_lr, cfg.weight_decay, store=strategy.store)
    loader = TokenLoader("synthetic", "train", SEQ, MICRO, seed=cfg.seed, rank=strategy.dp_rank, world_size=strategy.dp_world, device=d.device)
    accum = cfg.grad_accum(strategy.dp_world)
    losses = []
    for _ in range(STEPS):
        # (in the single-GPU run every rank trains the same replica on the same data, so the loss mean over ranks is the loss)
        losses.append(train_step(strategy, opt, loader, accum, cfg.grad_clip, AMP_DTYPES["bf16"])[0])
    torch.cuda.synchronize()
    del strategy, opt, loader
    gc.collect()
    torch.cuda.empty_cache()
    return losses


def main():
    d = parallel.init()
    world = d.world
    ok = check_collectives(d)
    say(f"COLLECTIVES world={world}: {'ok' if ok else 'MISMATCH'}")
    single = run_layout(d, "none", fake_single=True)
    say("single-GPU losses:", [round(x, 4) for x in single])
    layouts = [("ddp", {}), ("ddp+graph", {"parallel": "ddp", "cuda_graph": True}), ("fsdp", {}),
               ("fsdp, all-gather inside the QKV GEMM", {"parallel": "fsdp", "fsdp_gemm_gather": True}), ("tp", {})]
    if world >= 4:
        layouts.append(("fsdp_tp", {"tp_size": 2}))
    for name, extra in layouts:
        par = extra.pop("parallel", name)
        losses = run_layout(d, par, extra)
        worst = max(abs(a - b) for a, b in zip(losses, single))
        good = worst <= TOL and all(x == x for x in losses)
        ok &= good
        say(f"PARITY world={world} {name}: max |loss - single| = {worst:.4f} {'ok' if good else 'FAIL'}  {[round(x, 4) for x in losses]}")
        dist.barrier()
    # without gradient clipping the sharded AdamW step runs inside the reduce-scatter kernels
    single_nc = run_layout(d, "none", {"grad_clip": 0.0}, fake_single=True)
    for name, par in (("fsdp, update inside the reduce-scatter", "fsdp"), ("ddp, no clipping", "ddp")):
        losses = run_layout(d, par, {"grad_clip": 0.0})
        worst = max(abs(a - b) for a, b in zip(losses, single_nc))
        good = worst <= TOL and all(x == x for x in losses)
        ok &= good
        say(f"PARITY world={world} {name}: max |loss - single| = {worst:.4f} {'ok' if good else 'FAIL'}  {[round(x, 4) for x in losses]}")
        dist.barrier()
    flag = torch.tensor([0.0 if ok else 1.0], device=d.device)
    dist.all_reduce(flag)
    say("PARITY_OK" if flag.item() == 0 else "PARITY_FAILED")
    parallel.destroy()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
