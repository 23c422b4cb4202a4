"""Tensor parallel + sequence parallel (Megatron style) with vocab-parallel embedding and loss.

Layout, as in the reference (nanonemo/distributed/tp.py:33-66): ``wqkv`` / ``w_gu`` are column
parallel (each rank owns H/tp query heads, KVH/tp KV heads, d_ff/tp hidden units), ``wo`` /
``w_down`` row parallel, the tied embedding / head is sharded over the vocabulary, norm weights are
replicated; the residual stream, the norms and the residual adds hold 1/tp of the tokens per rank
(sequence parallel), with an all-gather entering attention / MLP / head and a reduce-scatter leaving
``wo`` / ``w_down``; the loss is computed on vocabulary shards (three small all-reduces: row max,
sum-exp, target logit) so full logits are never gathered.

Differences: the model is built from the same seed as a single-process model and then SLICED
(``shard_model_``), so initial weights match exactly; tokens are partitioned as contiguous chunks of
the flattened (B*T) token axis, which makes every gather / scatter a contiguous copy; the local
parameters live in a ``FlatParams`` store so clipping and AdamW are the fused flat kernels; and the
operators on local tensors (norm, RoPE, attention, SwiGLU, GEMMs) are the same sm100 kernels as on
one GPU — the reference has to force its ``torch`` norms and loss under TP (tp.py:37-38).
Degrees that do not divide the head counts (8 with 12 query / 4 KV heads) use rank PAIRS: the MLP, the vocabulary and the
norms are split ``tp`` ways as usual, the heads ``tp / 2`` ways; the two ranks of a pair hold the same ``wqkv`` / ``wo``
slices, attend over the first half (rank 0 of the pair) or the whole (rank 1) of every sequence and project only their own
half of the query rows, contributing zeros for the other half to the reduce-scatter; their weight gradients are summed inside
the pair. With ``comm="fused"`` (and the sm100 GEMM) the four block linears run as single kernels that do the
collective themselves (parallel/tp_fused.py: all-gather -> GEMM and GEMM -> reduce-scatter over peer
memory) and the embedding is one kernel that stores every owned row into its token owner's memory (csrc/comm.cu:
vp_embed_fwd_kernel / vp_embed_bwd_kernel); the head / loss collectives and the CPU path use torch.distributed.
"""

import torch
import torch.distributed as dist
import torch.nn.functional as F

from nanonemo_b200.parallel.strategy import LocalStrategy


# ----------------------------------------------------------------------------- collectives with autograd
class TPContext:
    def __init__(self, group, rank: int, world: int, device, fused_tp=None):
        self.group, self.rank, self.world, self.device = group, rank, world, torch.device(device)
        self.fused_tp = fused_tp  # parallel.tp_fused.FusedTP: linears whose collective runs inside the GEMM kernel
        self.B = self.T = 0
        self.gloo = self.device.type != "cuda"
        # attention layout (set_attention_layout): heads are split attn_world ways; when the heads do not divide by the
        # degree, consecutive PAIRS of ranks share a head group (same wqkv / wo slices) and split its query rows
        self.attn_world, self.attn_rank, self.pair, self.pair_pos, self.pair_group = world, rank, 1, 0, None

    def set_attention_layout(self, cfg, pair_group=None):
        self.attn_world, self.pair = attention_layout(cfg, self.world)
        self.attn_rank, self.pair_pos = self.rank // self.pair, self.rank % self.pair
        self.pair_group = pair_group
        if self.pair > 1 and pair_group is None:
            raise ValueError("a tensor-parallel degree that needs the pair split must be given the pair process group")

    # raw collectives on contiguous 2-D tensors, along dim 0
    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        out = torch.empty((x.shape[0] * self.world, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=self.group)
        return out

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        n = x.shape[0] // self.world
        if self.gloo:
            x = x.clone()
            dist.all_reduce(x, group=self.group)
            return x[self.rank * n:(self.rank + 1) * n].clone()
        out = torch.empty((n, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=self.group)
        return out

    def all_reduce(self, x: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        dist.all_reduce(x, op=op, group=self.group)
        return x

    # differentiable forms
    def gather_tokens(self, x):
        return _Gather.apply(x, self)

    def scatter_tokens(self, x):
        return _ReduceScatter.apply(x, self)


class _Gather(torch.autograd.Function):
    """all-gather along tokens; backward is the reduce-scatter of the gradient."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.all_gather(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.reduce_scatter(g), None


class _ReduceScatter(torch.autograd.Function):
    """reduce-scatter along tokens; backward is the all-gather of the gradient."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.reduce_scatter(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_gather(g), None


class _VocabParallelEmbedding(torch.autograd.Function):
    """Rows of the vocabulary shard this rank owns, zeros elsewhere, summed and scattered over tokens."""

    @staticmethod
    def forward(ctx, idx_flat, weight, tp, v0, out_dtype):
        V = weight.shape[0]
        ft = tp.fused_tp
        ctx.in_kernel = (ft is not None and weight.dtype == torch.float32 and weight.shape[1] % 8 == 0
                         and idx_flat.numel() // tp.world * weight.shape[1] <= ft.embed_stage.tensor.numel())
        if ctx.in_kernel:
            # one kernel: every rank stores the rows it owns straight into the token owners' memory (parallel/tp_fused.py)
            idx64 = idx_flat if idx_flat.dtype == torch.int64 else idx_flat.long()
            idx64 = idx64.contiguous()
            ctx.save_for_backward(idx64, weight)
            ctx.tp, ctx.v0 = tp, v0
            return ft.embed_rows(idx64, weight.detach().contiguous(), v0, out_dtype)
        local = idx_flat - v0
        mine = (local >= 0) & (local < V)
        rows = F.embedding(local.clamp(0, V - 1), weight).to(out_dtype)
        rows = rows * mine.unsqueeze(-1).to(rows.dtype)
        ctx.save_for_backward(local, mine, weight)
        ctx.tp = tp
        return tp.reduce_scatter(rows)

    @staticmethod
    def backward(ctx, g):
        if ctx.in_kernel:
            idx64, weight = ctx.saved_tensors
            main = getattr(weight, "_main_grad", None)
            target = main if main is not None and main.dtype == torch.float32 else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            ctx.tp.fused_tp.embed_grad(idx64, g.contiguous(), target, ctx.v0)
            if target is main:
                cb = getattr(weight, "_grad_ready_cb", None)
                if cb is not None:
                    cb(weight, True)
                return None, None, None, None, None
            return None, target.to(weight.dtype), None, None, None
        local, mine, weight = ctx.saved_tensors
        g_full = ctx.tp.all_gather(g).float() * mine.unsqueeze(-1)
        main = getattr(weight, "_main_grad", None)
        target = main if main is not None and main.dtype == torch.float32 else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        target.index_add_(0, local.clamp(0, weight.shape[0] - 1), g_full)
        if target is main:
            cb = getattr(weight, "_grad_ready_cb", None)
            if cb is not None:
                cb(weight, True)
            return None, None, None, None, None
        return None, target.to(weight.dtype), None, None, None


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross entropy over vocabulary shards: logits_local [N, V/tp]; targets are global ids."""

    @staticmethod
    def forward(ctx, logits, targets, tp, v0):
        lf = logits.float()
        m = tp.all_reduce(lf.max(dim=-1).values, dist.ReduceOp.MAX)
        e = torch.exp(lf - m.unsqueeze(-1))
        s = tp.all_reduce(e.sum(dim=-1))
        local = targets - v0
        mine = (local >= 0) & (local < lf.shape[1])
        tl = lf.gather(1, local.clamp(0, lf.shape[1] - 1).unsqueeze(1)).squeeze(1) * mine
        tl = tp.all_reduce(tl)
        loss = (m + torch.log(s) - tl).mean()
        ctx.save_for_backward(e, s, local, mine)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        e, s, local, mine = ctx.saved_tensors
        N = e.shape[0]
        grad = e / s.unsqueeze(-1)
        rows = torch.arange(N, device=e.device)[mine]
        grad[rows, local[mine]] -= 1.0
        return (grad * (g / N)).to(ctx.dtype), None, None, None


# ----------------------------------------------------------------------------- model surgery
def attention_layout(cfg, tp: int):
    """(ways the heads are split, ranks per head group). Head-aligned when the degree divides both head counts (12 query /
    4 KV heads: 1, 2, 4); otherwise pairs of ranks share a head group and split its query rows (12 / 4 heads at degree 8:
    4 groups x 2) — the layout the reference refuses (nanonemo/distributed/tp.py:35-36)."""
    if cfg.n_heads % tp == 0 and cfg.n_kv_heads % tp == 0:
        return tp, 1
    if tp % 2 == 0 and cfg.n_heads % (tp // 2) == 0 and cfg.n_kv_heads % (tp // 2) == 0:
        return tp // 2, 2
    raise ValueError(f"tensor parallel degree {tp} fits neither n_heads={cfg.n_heads} / n_kv_heads={cfg.n_kv_heads} "
                     f"head-aligned nor with rank pairs sharing a head group")


def check_divisible(cfg, tp: int):
    attention_layout(cfg, tp)
    if cfg.d_ff % tp or cfg.vocab_size % tp:
        raise ValueError(f"tensor parallel degree {tp} must divide d_ff={cfg.d_ff} and vocab_size={cfg.vocab_size}")


@torch.no_grad()
def shard_model_(model, tp: TPContext):
    """Slice a fully initialised model in place to this rank's tensor-parallel shard."""
    cfg, r, W = model.cfg, tp.rank, tp.world
    check_divisible(cfg, W)
    if (tp.attn_world, tp.pair) != attention_layout(cfg, W):
        tp.set_attention_layout(cfg, tp.pair_group)
    ar, aw = tp.attn_rank, tp.attn_world
    hd = cfg.head_dim
    Hl, KVl, Fl, Vl = cfg.n_heads // aw, cfg.n_kv_heads // aw, cfg.d_ff // W, cfg.vocab_size // W
    for block in model.blocks:
        a, m = block.attn, block.mlp
        wq, wk, wv = a.split_qkv()
        a.wqkv.weight.data = torch.cat((wq[ar * Hl * hd:(ar + 1) * Hl * hd], wk[ar * KVl * hd:(ar + 1) * KVl * hd],
                                        wv[ar * KVl * hd:(ar + 1) * KVl * hd])).contiguous()
        a.wo.weight.data = a.wo.weight[:, ar * Hl * hd:(ar + 1) * Hl * hd].contiguous()
        a.n_heads, a.n_kv_heads, a.q_dim, a.kv_dim = Hl, KVl, Hl * hd, KVl * hd
        wg, wu = m.split_gu()
        m.w_gu.weight.data = torch.cat((wg[r * Fl:(r + 1) * Fl], wu[r * Fl:(r + 1) * Fl])).contiguous()
        m.w_down.weight.data = m.w_down.weight[:, r * Fl:(r + 1) * Fl].contiguous()
        m.d_ff = Fl
        a.tp = m.tp = tp
    model.tok_emb.weight.data = model.tok_emb.weight[r * Vl:(r + 1) * Vl].contiguous()
    model.tp, model.vocab_start = tp, r * Vl
    model._mark_gradient_paths()  # the vocabulary-parallel embedding writes its gradient directly: re-derive who reports the tied weight
    return model


SHARD_DIMS = {"attn.wqkv.weight": "qkv", "attn.wo.weight": 1, "mlp.w_gu.weight": "gu", "mlp.w_down.weight": 1,
              "tok_emb.weight": 0}


def shard_rule(name: str):
    for key, rule in SHARD_DIMS.items():
        if name.endswith(key):
            return rule
    return None  # replicated (norm weights)


class TPStrategy(LocalStrategy):
    name = "tp"
    sharded_grads = True

    def __init__(self, model, tp: TPContext, store, step_model=None, dp_group=None):
        super().__init__(model, store, step_model)
        self.tp = tp
        self.replicated = [p for n, p in model.named_parameters() if shard_rule(n) is None]
        # rank pairs that share a head group hold identical wqkv / wo slices, each with the gradient of its own query rows
        self.duplicated = [p for n, p in model.named_parameters() if tp.pair > 1 and is_attention_weight(n)]
        self.dp_rank, self.dp_world = 0, 1  # every TP rank reads the same batch: one data-parallel replica

    def finish_grads(self):
        # norm weights saw only this rank's tokens: sum their gradients over the TP group
        if self.replicated:
            flat = torch.cat([p._main_grad.reshape(-1) if hasattr(p, "_main_grad") else p.grad.reshape(-1) for p in self.replicated])
            self.tp.all_reduce(flat)
            o = 0
            for p in self.replicated:
                g = p._main_grad if hasattr(p, "_main_grad") else p.grad
                g.copy_(flat[o:o + p.numel()].view(p.shape))
                o += p.numel()
        for p in self.duplicated:  # sum the two row halves' contributions: both ranks of a pair end with the same gradient
            g = p._main_grad if hasattr(p, "_main_grad") else p.grad
            dist.all_reduce(g, group=self.tp.pair_group)

    def status_words(self) -> list:
        words = super().status_words()
        ft = self.tp.fused_tp
        if ft is not None:
            words += [ft.fg.comm_status, ft.comm.status]
        return words

    def status_owners(self) -> list:
        ft = self.tp.fused_tp
        return [ft.fg, ft.comm] if ft is not None else []

    def global_sumsq(self):
        total = self.store.grad_sumsq()
        zero = torch.zeros((), device=total.device)
        rep = sum((p._main_grad.float().pow(2).sum() for p in self.replicated), zero)
        dup = sum((p._main_grad.float().pow(2).sum() for p in self.duplicated), zero)  # held by `pair` ranks: count once
        sharded = self.tp.all_reduce((total - rep - dup + dup / self.tp.pair).reshape(1).clone()).reshape(())
        return sharded + rep

    # checkpoint state: gather the shards back to full tensors
    def _full(self, name, local):
        return tp_full_tensor(name, local, self.tp, self.model.cfg)

    def _local(self, name, full):
        return tp_local_slice(name, full, self.tp, self.model.cfg)

    def checkpoint_names(self) -> list:
        return [(n, tp_full_shape(n, shape, self.tp, self.model.cfg)) for n, shape in super().checkpoint_names()]

    def checkpoint_tensors(self, opt, kind: str):
        for n, local in super().checkpoint_tensors(opt, kind):
            yield n, self._full(n, local)

    def restore_tensor(self, opt, kind: str, name: str, full: torch.Tensor) -> None:
        dev = next(self.model.parameters()).device
        super().restore_tensor(opt, kind, name, self._local(name, full.to(dev)))


def is_attention_weight(name: str) -> bool:
    return name.endswith("attn.wqkv.weight") or name.endswith("attn.wo.weight")


def tp_full_tensor(name, local, tp, cfg):
    """All-gather a tensor-parallel shard of parameter `name` back to the full tensor."""
    rule = shard_rule(name)
    if rule is None:
        return local.detach().clone()
    parts = [torch.empty_like(local) for _ in range(tp.world)]
    dist.all_gather(parts, local.detach().contiguous(), group=tp.group)
    hd, W = cfg.head_dim, tp.world
    if is_attention_weight(name):
        parts, W = parts[::tp.pair], tp.attn_world  # one copy per head group
    if rule == "qkv":
        q, kv = cfg.n_heads // W * hd, cfg.n_kv_heads // W * hd
        return torch.cat([p[:q] for p in parts] + [p[q:q + kv] for p in parts] + [p[q + kv:] for p in parts])
    if rule == "gu":
        f = cfg.d_ff // W
        return torch.cat([p[:f] for p in parts] + [p[f:] for p in parts])
    return torch.cat(parts, dim=rule)


def tp_full_shape(name, local_shape, tp, cfg) -> tuple:
    """Shape of the full tensor whose tensor-parallel shard has `local_shape`."""
    rule = shard_rule(name)
    if rule is None:
        return tuple(local_shape)
    W = tp.attn_world if is_attention_weight(name) else tp.world
    dim = 0 if rule in ("qkv", "gu") else rule
    full = list(local_shape)
    full[dim] *= W
    return tuple(full)


def tp_local_slice(name, full, tp, cfg):
    """This rank's tensor-parallel shard of the full tensor of parameter `name`."""
    rule = shard_rule(name)
    if rule is None:
        return full
    r, W, hd = tp.rank, tp.world, cfg.head_dim
    if is_attention_weight(name):
        r, W = tp.attn_rank, tp.attn_world
    if rule == "qkv":
        Q, KV = cfg.n_heads * hd, cfg.n_kv_heads * hd
        q, kv = Q // W, KV // W
        return torch.cat((full[r * q:(r + 1) * q], full[Q + r * kv:Q + (r + 1) * kv], full[Q + KV + r * kv:Q + KV + (r + 1) * kv]))
    if rule == "gu":
        Fd, f = cfg.d_ff, cfg.d_ff // W
        return torch.cat((full[r * f:(r + 1) * f], full[Fd + r * f:Fd + (r + 1) * f]))
    n = full.shape[rule] // W
    return full.narrow(rule, r * n, n)


def make_pair_group(tp_rank_lists, pair: int):
    """Process groups of consecutive `pair` ranks inside every tensor-parallel group; every rank of the world creates every
    group, in the same order, and gets back the one it belongs to."""
    mine, me = None, dist.get_rank()
    for ranks in tp_rank_lists:
        for i in range(0, len(ranks), pair):
            sub = ranks[i:i + pair]
            grp = dist.new_group(sub)
            if me in sub:
                mine = grp
    return mine


def _maybe_fuse(tp, model_cfg, cfg, d, group):
    from nanonemo_b200.parallel.symm import fused_available

    tokens = cfg.micro_batch * cfg.seq_len
    # (under the rank-pair layout only the MLP uses the fused linears: the pair split of attention gathers the whole sequence
    # and scatters half-empty rows, which the unfused path handles; see models/layers.py)
    if (fused_available(d, cfg.comm) and model_cfg.resolved().linear_impl == "sm100" and cfg.precision in ("bf16", "fp16")
            and tokens % (128 * tp.world) == 0):
        from nanonemo_b200.parallel.tp_fused import FusedTP

        dt = torch.bfloat16 if cfg.precision == "bf16" else torch.float16
        tp.fused_tp = FusedTP(d.device, group, tp.rank, tp.world, tokens, model_cfg.d_model, dt)


def build_tp(model_cfg, cfg, d):
    """parallel=tp: the whole world is one tensor-parallel group. parallel=fsdp_tp: a 2-D mesh, consecutive
    groups of tp_size ranks are tensor parallel and the parameters each of them holds are fully sharded
    over the world / tp_size data-parallel ranks with the same position in their group."""
    from nanonemo_b200.parallel.flat import FlatParams
    from nanonemo_b200.train.trainer import build_model, shadow_dtype

    world, rank = dist.get_world_size(), dist.get_rank()
    if cfg.parallel == "tp":
        if (cfg.tp_size or world) != world:
            raise ValueError("parallel=tp uses the whole world as the tensor-parallel group; use fsdp_tp for a 2-D mesh")
        tp = TPContext(dist.group.WORLD, rank, world, d.device)
        _, pair = attention_layout(model_cfg, world)
        tp.set_attention_layout(model_cfg, make_pair_group([list(range(world))], pair) if pair > 1 else None)
        model, step_model = build_model(model_cfg, cfg, d.device)
        shard_model_(model, tp)
        _maybe_fuse(tp, model_cfg, cfg, d, dist.group.WORLD)
        store = FlatParams(model, d.device, shadow_dtype(model_cfg, cfg))
        return TPStrategy(model, tp, store, step_model)

    tps = cfg.tp_size
    if world % tps:
        raise ValueError(f"tp_size {tps} does not divide the world size {world}")
    tp_group = dp_group = None
    for g in range(world // tps):  # every rank creates every group, in the same order
        ranks = list(range(g * tps, (g + 1) * tps))
        grp = dist.new_group(ranks)
        if rank in ranks:
            tp_group = grp
    for i in range(tps):
        ranks = list(range(i, world, tps))
        grp = dist.new_group(ranks)
        if rank in ranks:
            dp_group = grp
    tp = TPContext(tp_group, rank % tps, tps, d.device)
    if attention_layout(model_cfg, tps)[1] > 1:
        raise ValueError(f"tp_size {tps} needs rank pairs to share a head group, which the 2-D fsdp_tp mesh does not support; "
                         "use parallel=tp or a head-aligned tp_size")
    model, step_model = build_model(model_cfg, cfg, d.device)
    shard_model_(model, tp)
    _maybe_fuse(tp, model_cfg, cfg, d, tp_group)
    from nanonemo_b200.parallel.fsdp import FSDPTPStrategy

    pd = cfg.fsdp_param_dtype
    if pd == "fp32" and model_cfg.uses_sm100("linear_impl") and cfg.precision in ("bf16", "fp8"):
        pd = "bf16"
    return FSDPTPStrategy(model, d, tp, pd, cfg.fsdp_reshard_after_forward, cfg.fsdp_prefetch, cfg.comm, group=dp_group,
                          step_model=step_model, precision=cfg.precision)
