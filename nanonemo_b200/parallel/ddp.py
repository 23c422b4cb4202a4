"""Data parallel: bucketed gradient all-reduce overlapped with backward, on the flat gradient buffer.

What torch DDP's C++ reducer does for the reference (nanonemo/distributed/ddp.py:14-16: fp32 grads
bucketed by ``bucket_cap_mb``, all-reduced as they become ready, ``no_sync`` on all but the last
micro-batch) is done here on index ranges of ``FlatParams.grad``:

* parameters are walked in reverse registration order and cut into buckets of ``bucket_cap_mb``; as
  flat offsets follow registration order each bucket is one contiguous range of the buffer;
* a gradient is "ready" when autograd has accumulated it (post-accumulate hook) or when the sm100
  linear backward, which accumulates straight into the flat buffer, says so;
* when the last micro-batch completes a bucket, the bucket is reduced on a side stream so it
  overlaps the rest of backward. With ``comm="fused"`` (CUDA, built library) the reduction is the
  hand-written two-shot all-reduce kernel over NVLink peer pointers, which also applies the
  ``1 / world`` average and accumulates the squared norm of the reduced slice for clipping;
  otherwise it is ``dist.all_reduce`` (NCCL, or gloo on CPU) followed by the average;
* buckets are always launched in bucket order on every rank, so ranks never disagree on the order
  of collectives;
* the fused kernel keeps its epoch counters in device memory, so with ``cuda_graph: true`` the hooks'
  launches are captured together with forward and backward and the whole micro-batch, collectives
  included, replays as one graph;
* the squared norm of the reduced gradient comes out of the all-reduce kernels themselves (a table of
  per-block partial sums that every rank adds up in the same order), so clipping costs no pass over
  the gradient and every rank computes bit-identical clip coefficients.

Gradients are always views into the bucket buffer, which is what ``ddp_grad_as_bucket_view``
asks for in the reference; the knob is accepted and has no further effect.
"""

from contextlib import contextmanager

import torch
import torch.distributed as dist

from nanonemo_b200.parallel.flat import FlatParams
from nanonemo_b200.parallel.strategy import LocalStrategy


class Bucket:
    __slots__ = ("lo", "hi", "params", "pending", "work")

    def __init__(self):
        self.lo, self.hi, self.params, self.pending, self.work = None, None, [], 0, None


def build_buckets(store: FlatParams, cap_bytes: float) -> list[Bucket]:
    buckets, cur = [], Bucket()
    for p in reversed(store.params):
        lo, hi = store.range_of(p)
        if cur.params and (cur.hi - lo) * 4 > cap_bytes:
            buckets.append(cur)
            cur = Bucket()
        cur.lo = lo
        cur.hi = hi if cur.hi is None else cur.hi
        cur.params.append(p)
    if cur.params:
        buckets.append(cur)
    buckets[0].hi = store.numel  # the tail padding rides with the first (last-registered) bucket
    return buckets


class DDPStrategy(LocalStrategy):
    name = "ddp"

    def __init__(self, model, d, store: FlatParams, bucket_cap_mb: float = 25.0, comm: str = "auto",
                 group=None, symm=None, step_model=None):
        super().__init__(model, store, step_model)
        self.group = group
        self.dp_rank, self.dp_world = dist.get_rank(group), dist.get_world_size(group)
        self.buckets = build_buckets(store, bucket_cap_mb * 2**20)
        self._bucket_of = {id(p): b for b in self.buckets for p in b.params}
        self._sync = True
        self._next = 0  # next bucket to launch (strict order)
        self._ready = [False] * len(self.buckets)
        self.symm = symm  # SymmetricAllReduce over store.grad, or None -> torch.distributed
        self.fused = symm is not None
        self._cuda = store.device.type == "cuda"
        self._comm_stream = torch.cuda.Stream(device=store.device) if self._cuda else None
        self._done = False  # finish_grads() already ran for the current step
        for p in store.params:
            p.register_post_accumulate_grad_hook(self._on_grad)
            p._grad_ready_cb = self._on_grad
        self._reset()
        self.check_replicas()

    def check_replicas(self):
        """Every rank built the model from the same seed; verify instead of broadcasting 457 MB."""
        s = self.store.master.double().sum().reshape(1)
        both = torch.cat([s, -s])
        dist.all_reduce(both, op=dist.ReduceOp.MAX, group=self.group)
        if not torch.allclose(both[0], -both[1], rtol=0, atol=0):
            for p in self.store.params:  # fall back to the reference behaviour: rank 0's weights win
                dist.broadcast(p.data, src=dist.get_global_rank(self.group, 0) if self.group else 0, group=self.group)
            self.store.refresh_shadow()

    def _reset(self):
        for b in self.buckets:
            b.pending, b.work = len(b.params), None
        self._next = 0
        self._ready = [False] * len(self.buckets)
        self._done = False

    @contextmanager
    def _no_sync(self):
        self._sync = False
        try:
            yield
        finally:
            self._sync = True

    def sync_ctx(self, last: bool):
        if last:
            self._reset()
            return super().sync_ctx(last)
        return self._no_sync()

    # -- gradient-ready path
    def _on_grad(self, p, manual: bool = False):
        # Parameters whose gradient is written straight into the flat buffer by an sm100 backward
        # (p._manual_ready) report readiness themselves; autograd's hook for them is ignored.
        if not self._sync or getattr(p, "_manual_ready", False) != manual:  # one reporting channel per parameter
            return
        b = self._bucket_of[id(p)]
        b.pending -= 1
        if b.pending == 0:
            self._ready[self.buckets.index(b)] = True
            while self._next < len(self.buckets) and self._ready[self._next]:
                self._launch(self.buckets[self._next])
                self._next += 1

    def _launch(self, b: Bucket):
        view = self.store.grad[b.lo:b.hi]
        if self.fused:
            ev = torch.cuda.Event()
            ev.record()
            self._comm_stream.wait_event(ev)
            with torch.cuda.stream(self._comm_stream):
                self.symm.all_reduce_(b.lo, b.hi, scale=1.0 / self.dp_world, bucket=self.buckets.index(b))
            self.launches += 1
            b.work = True
        elif self._cuda:
            ev = torch.cuda.Event()
            ev.record()
            self._comm_stream.wait_event(ev)
            with torch.cuda.stream(self._comm_stream):
                dist.all_reduce(view, group=self.group)
                view.mul_(1.0 / self.dp_world)
            b.work = True
        else:
            b.work = dist.all_reduce(view, group=self.group, async_op=True)

    def finish_grads(self):
        if self._done:
            return
        # Any bucket whose parameters never produced a gradient this step is still reduced (zeros).
        while self._next < len(self.buckets):
            self._launch(self.buckets[self._next])
            self._next += 1
        if self._cuda:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        else:
            for b in self.buckets:
                if b.work is not None and b.work is not True:
                    b.work.wait()
                self.store.grad[b.lo:b.hi].mul_(1.0 / self.dp_world)
        self._reset()
        self._done = True

    def after_graph_replay(self):
        self._done = True  # the replayed graph contained every bucket's all-reduce and the join of the side stream

    def global_sumsq(self):
        # Every rank holds the same averaged gradient after the all-reduce. The fused kernels left the squared norm of every
        # reduced slice in a table that is identical on all ranks; otherwise one local pass over the gradient gives it.
        if self.fused:
            return self.symm.norm_sq(len(self.buckets))
        return self.store.grad_sumsq()

    def status_words(self) -> list:
        words = super().status_words()
        if self.fused:
            words.append(self.symm.status)
        return words

    def status_owners(self) -> list:
        return [self.symm] if self.fused else []
