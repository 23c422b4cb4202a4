"""Symmetric-memory layer: buffers mapped into every peer GPU, and the collectives written on them.

``torch.distributed._symmetric_memory`` is used only as the allocator and handshake (it exchanges
the cuMem handles and gives each rank the peers' device pointers, and the NVLS multicast address
when the driver exposes one). The data movement is this framework's own kernels (csrc/comm.cu):
peer loads and stores issued from inside the kernel, synchronised by epoch-numbered flags in a
second symmetric buffer with system-scope release/acquire, every wait bounded in time (on expiry the
kernel records {code, rank, peer, block} in a status word and returns; the training step reads that word
together with its loss and raises on the host, see ``parallel.strategy.LocalStrategy.status_words``).

The reference has no counterpart: its collectives are NCCL calls made by torch DDP / FSDP2 / DTensor
(nanonemo/distributed/*.py).
"""

import ctypes
import os

import torch
import torch.distributed as dist

STATUS_WORDS = 8


def fused_available(d, comm: str) -> bool:
    if comm == "nccl" or not str(d.device).startswith("cuda"):
        return False
    from nanonemo_b200.ops import _lib

    ok = _lib.available()
    if comm == "fused" and not ok:
        raise RuntimeError("comm=fused needs a CUDA device and the built kernel library")
    return ok


class SymmetricBuffer:
    """A tensor allocated in symmetric memory plus the peers' pointers to it."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group=group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.ptr_array = (ctypes.c_void_p * 16)(*self.peer_ptrs)


MAX_NORM_BUCKETS = 256  # rows of the partial-norm table (gradient buckets per optimizer step)


def comm_timeout_s() -> float:
    """Time limit of every cross-GPU wait inside the collective kernels (seconds; NANONEMO_COMM_TIMEOUT_S, default 30)."""
    return float(os.environ.get("NANONEMO_COMM_TIMEOUT_S", "30"))


class SymmetricComm:
    """Launcher of the collective kernels (csrc/comm.cu) for one group: owns the symmetric flag buffer, the per-block
    epoch counters (device memory: the launch arguments never change, so the collectives replay from a CUDA graph) and
    the status words the kernels write when a bounded wait runs out."""

    def __init__(self, device, group, rank: int, world: int, blocks: int | None = None):
        from nanonemo_b200.ops import _lib

        self.rank, self.world, self.group = rank, world, group
        # two light blocks per SM (128 threads, <= 85 registers each: csrc/comm.cu comm_threads()): one always fits beside whatever
        # compute kernel is resident, both fit beside the plain GEMMs
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.blocks = blocks or int(os.environ.get("NANONEMO_COMM_BLOCKS", str(2 * sms)))
        words = _lib.lib().nnb_comm_flag_words(self.blocks)
        self.flags = SymmetricBuffer(words, torch.int32, device, group)
        self.flags.tensor.zero_()
        self.epochs = torch.zeros(self.blocks, dtype=torch.int32, device=device)
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)
        self.timeout_s = comm_timeout_s()
        self.norm_parts = None  # SymmetricBuffer [MAX_NORM_BUCKETS, world, blocks] once enable_norm_parts() was called
        self._norm_out = None
        self._null_ptrs = (ctypes.c_void_p * 16)()
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def enable_norm_parts(self):
        """Allocate the table the all-reduce kernels fill with the squared norm of every reduced slice."""
        dev = self.flags.tensor.device
        self.norm_parts = SymmetricBuffer(MAX_NORM_BUCKETS * self.world * self.blocks, torch.float32, dev, self.group)
        self.norm_parts.tensor.zero_()
        self._norm_out = torch.zeros(1, dtype=torch.float32, device=dev)
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)

    def all_reduce_(self, data: "SymmetricBuffer", lo: int, hi: int, scale: float, multimem: bool = False, bucket: int = -1):
        """In place: data[lo:hi] = scale * sum over ranks. With `bucket` >= 0 (and enable_norm_parts()) the kernel also
        leaves the squared norm of every reduced slice in row `bucket` of the partial-norm table of every rank."""
        from nanonemo_b200.ops import _lib

        _lib.call("nnb_allreduce_f32", data.ptr_array, self.flags.ptr_array, self._norm_args(bucket),
                  ctypes.c_void_p(data.multicast_ptr if multimem else 0), _lib.ptr(self.status), _lib.ptr(self.epochs),
                  _lib.i32(self.rank), _lib.i32(self.world), _lib.i64(lo), _lib.i64(hi - lo), _lib.f32(scale),
                  _lib.i32(max(bucket, 0)), _lib.i32(self.blocks), ctypes.c_double(self.timeout_s),
                  ctypes.c_void_p(_lib.stream_ptr()))

    def norm_sq(self, n_buckets: int) -> torch.Tensor:
        """Sum of the partial-norm rows [0, n_buckets): the squared global norm of the reduced gradient, added in a
        fixed order (every rank holds the same table, so every rank gets the same bits). 0-dim device tensor."""
        from nanonemo_b200.ops import _lib

        _lib.call("nnb_sumsq_combine", _lib.ptr(self.norm_parts.tensor), _lib.i64(n_buckets * self.world * self.blocks),
                  _lib.ptr(self._norm_out), ctypes.c_void_p(_lib.stream_ptr()))
        return self._norm_out[0]

    def _norm_args(self, bucket: int):
        with_norm = bucket >= 0 and self.norm_parts is not None
        assert bucket < MAX_NORM_BUCKETS
        return self.norm_parts.ptr_array if with_norm else self._null_ptrs

    def reduce_scatter(self, data: "SymmetricBuffer", out: torch.Tensor, sumsq: torch.Tensor | None, lo: int, per: int,
                       scale: float, bucket: int = -1):
        """out[i] = scale * sum over ranks of data[lo + rank * per + i]; sumsq += sum(out ** 2) when given; with
        `bucket` >= 0 the squared norm also goes to row `bucket` of every rank's norm table (see norm_sq)."""
        from nanonemo_b200.ops import _lib

        _lib.call("nnb_reduce_scatter_f32", data.ptr_array, self.flags.ptr_array, self._norm_args(bucket), _lib.ptr(out),
                  _lib.ptr(sumsq), _lib.ptr(self.status), _lib.ptr(self.epochs), _lib.i32(self.rank), _lib.i32(self.world),
                  _lib.i64(lo), _lib.i64(per), _lib.f32(scale), _lib.i32(max(bucket, 0)), _lib.i32(self.blocks),
                  ctypes.c_double(self.timeout_s), ctypes.c_void_p(_lib.stream_ptr()))

    def reduce_scatter_adamw(self, data: "SymmetricBuffer", p, m, v, wire, decay_flags, lo: int, per: int, scale: float, bucket: int,
                             *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int):
        """Gradient reduce-scatter of one unit whose epilogue applies AdamW to this rank's shard (p, m, v: fp32 [per];
        wire: 16-bit copy or None). For training without clipping; the reduced gradient is never stored."""
        from nanonemo_b200.ops import _lib

        code = {torch.bfloat16: 1, torch.float16: 2}[wire.dtype] if wire is not None else 1
        _lib.call("nnb_reduce_scatter_adamw", data.ptr_array, self.flags.ptr_array, self._norm_args(bucket), _lib.ptr(p), _lib.ptr(m),
                  _lib.ptr(v), _lib.ptr(wire), _lib.ptr(decay_flags), _lib.ptr(self.status), _lib.ptr(self.epochs), _lib.i32(self.rank),
                  _lib.i32(self.world), _lib.i64(lo), _lib.i64(per), _lib.f32(scale), _lib.i32(max(bucket, 0)), _lib.i32(self.blocks),
                  ctypes.c_double(self.timeout_s), _lib.f32(lr), _lib.f32(beta1), _lib.f32(beta2), _lib.f32(eps), _lib.f32(weight_decay),
                  _lib.i32(step), _lib.i32(code), ctypes.c_void_p(_lib.stream_ptr()))

    def all_gather(self, shards: "SymmetricBuffer", full: torch.Tensor, src_off_bytes: int, per_bytes: int):
        """full[r * per : (r + 1) * per] = rank r's bytes [src_off, src_off + per) of `shards`."""
        from nanonemo_b200.ops import _lib

        _lib.call("nnb_allgather_bytes", shards.ptr_array, self.flags.ptr_array, _lib.ptr(full), _lib.ptr(self.status),
                  _lib.ptr(self.epochs), _lib.i32(self.rank), _lib.i32(self.world), _lib.i64(src_off_bytes),
                  _lib.i64(per_bytes), _lib.i32(self.blocks), ctypes.c_double(self.timeout_s),
                  ctypes.c_void_p(_lib.stream_ptr()))

    def peer_fetch(self, data: "SymmetricBuffer", items: torch.Tensor, n_items: int):
        """One launch copies `n_items` small ranges from the ranks that own them into local memory. `items`: device int64
        [n_items, 4] rows (src_off bytes, bytes, destination address, src_rank); everything 16-byte aligned."""
        from nanonemo_b200.ops import _lib

        _lib.call("nnb_peer_fetch", data.ptr_array, self.flags.ptr_array, _lib.ptr(items), _lib.i32(n_items), _lib.ptr(self.status),
                  _lib.ptr(self.epochs), _lib.i32(self.rank), _lib.i32(self.world), _lib.i32(self.blocks),
                  ctypes.c_double(self.timeout_s), ctypes.c_void_p(_lib.stream_ptr()))

    def vp_embedding(self, stage: "SymmetricBuffer", idx: torch.Tensor, rows: torch.Tensor, table: torch.Tensor, v0: int, backward: bool):
        """Vocabulary-parallel embedding over this group (csrc/comm.cu: vp_embed_fwd_kernel / vp_embed_bwd_kernel). idx: all
        world * per token ids (int64); table: this rank's fp32 rows [v0, v0 + V) of the weight (forward) or of its gradient
        (backward, added into); rows: this rank's [per, D] output (forward) or incoming gradient (backward). `stage`: a
        symmetric buffer of at least per * D elements of rows.dtype, free between calls."""
        from nanonemo_b200.ops import _lib

        per, D = rows.shape
        assert idx.numel() == per * self.world and idx.dtype == torch.int64 and table.dtype == torch.float32
        assert stage.tensor.numel() * stage.tensor.element_size() >= per * D * rows.element_size()
        _lib.call("nnb_vp_embedding_bwd" if backward else "nnb_vp_embedding_fwd", stage.ptr_array, self.flags.ptr_array, _lib.ptr(idx),
                  _lib.ptr(rows if backward else table), _lib.ptr(table if backward else rows), _lib.i64(per), _lib.i32(D), _lib.i64(v0),
                  _lib.i64(table.shape[0]), _lib.i32({torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[rows.dtype]),
                  _lib.ptr(self.status), _lib.ptr(self.epochs), _lib.i32(self.rank), _lib.i32(self.world), _lib.i32(self.blocks),
                  ctypes.c_double(self.timeout_s), ctypes.c_void_p(_lib.stream_ptr()))

    def check_status(self):
        st = self.status.tolist()
        if st[0] != 0:
            self.status.zero_()
            raise RuntimeError(f"fused collective gave up waiting: code={st[0]} rank={st[1]} peer={st[2]} "
                               f"block={st[3]} epoch={st[4]}")


class SymmetricAllReduce:
    """In-place two-shot all-reduce (+ scale, + squared norm of the result) over ranges of one symmetric fp32 buffer."""

    def __init__(self, data: SymmetricBuffer, group=None, with_norm: bool = True):
        self.data = data
        self.comm = SymmetricComm(data.tensor.device, group, data.rank, data.world)
        if with_norm:
            self.comm.enable_norm_parts()
        # NVSwitch multicast (multimem.ld_reduce / multimem.st): the switch does the sum, so a rank moves the data once instead of
        # 2 (N - 1) / N times. Measured for the 435 MiB gradient: 2 ranks 1.13 vs 0.71 ms (plain peer loads win: a single peer
        # load already is the whole reduction), 4 ranks 1.03 vs 1.05 ms, 8 ranks 0.99 vs 1.28 ms (NCCL: 1.15 ms). So it is used
        # from 8 ranks up (NANONEMO_MULTIMEM=1 / 0 forces it on / off), and only after a small all-reduce through the multicast
        # address has given the exact expected values on every rank.
        want = os.environ.get("NANONEMO_MULTIMEM", "auto")
        self.use_multimem = (bool(data.multicast_ptr) and (want == "1" or (want == "auto" and data.world >= 8))
                             and self._multicast_gives_exact_sums(group))

    def all_reduce_(self, lo: int, hi: int, scale: float, bucket: int = -1):
        self.comm.all_reduce_(self.data, lo, hi, scale, self.use_multimem, bucket)

    def _multicast_gives_exact_sums(self, group) -> bool:
        """One all-reduce of the buffer's first elements through the multicast address, on small integers (exact in any order);
        the elements are put back afterwards. False on any rank -> False on all (the plain peer-load path is used)."""
        t, world, rank = self.data.tensor, self.data.world, self.data.rank
        n = min(t.numel(), 4096 * world) // (4 * world) * (4 * world)
        if n == 0:
            return False
        keep = t[:n].clone()
        base = (torch.arange(n, device=t.device) % 13).float()
        t[:n] = base + rank
        torch.cuda.synchronize(t.device)
        dist.barrier(group)
        self.comm.all_reduce_(self.data, 0, n, 1.0, True, -1)
        good = torch.equal(t[:n], base * world + sum(range(world))) and int(self.comm.status[0].item()) == 0
        self.comm.status.zero_()
        torch.cuda.synchronize(t.device)
        dist.barrier(group)
        t[:n] = keep
        flag = torch.tensor([1 if good else 0], device=t.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        return bool(flag.item())

    def norm_sq(self, n_buckets: int) -> torch.Tensor:
        return self.comm.norm_sq(n_buckets)

    @property
    def status(self) -> torch.Tensor:
        return self.comm.status

    def check_status(self):
        self.comm.check_status()


def make_grad_allreduce(d, comm: str, group=None):
    """Returns (grad_alloc, finish): `grad_alloc(numel)` allocates the flat gradient buffer (in
    symmetric memory when the fused path is on), `finish(store)` returns the SymmetricAllReduce
    bound to it, or None when gradients are reduced with torch.distributed."""
    if not fused_available(d, comm):
        return None, lambda store: None
    box = {}

    def grad_alloc(numel: int):
        box["buf"] = SymmetricBuffer(numel, torch.float32, d.device, group)
        return box["buf"].tensor

    return grad_alloc, lambda store: SymmetricAllReduce(box["buf"], group)
