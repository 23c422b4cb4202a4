"""NanoNemo: Llama-style decoder-only transformer (pre-norm RMSNorm, RoPE, SwiGLU, GQA, tied head).

Behavioural reference: nanonemo/model/model.py:13-64 (init scheme, tied head, non-persistent RoPE
buffers, ``forward(idx, targets) -> (logits, loss)``, ``num_params``).
"""

import math

import torch
import torch.nn.functional as F
from torch import nn

from nanonemo_b200 import ops
from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.layers import AddRMSNorm, Block, Linear, rope_cache


class NanoNemo(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        r = cfg.resolved()
        self.tok_emb = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.norm_out = AddRMSNorm(cfg.d_model, cfg.norm_eps, r.norm_kernel)
        # The head stays a bf16 GEMM under mxfp8 (as the reference keeps lm_head out of its FP8 linears).
        self.lm_head = Linear(cfg.d_model, cfg.vocab_size, "sm100" if cfg.uses_sm100("linear_impl") else "torch")
        self.lm_head.weight = self.tok_emb.weight  # tied input/output embedding
        self.loss_impl, self.embed_impl = r.loss_kernel, r.embed_kernel
        self.tp, self.vocab_start = None, 0  # set by parallel.tp.shard_model_

        cos, sin = rope_cache(cfg.head_dim, cfg.max_seq_len, cfg.rope_base)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)
        self.reset_parameters()
        self._mark_gradient_paths()

    def _mark_gradient_paths(self):
        """Tell the gradient-ready bookkeeping (parallel/ddp.py) which parameters get their gradient
        written straight into the flat buffer by an sm100 backward (`_manual_ready`), and that the
        tied embedding/head weight is complete only after the embedding backward (`_tied_embedding`)."""
        w = self.tok_emb.weight
        w._tied_embedding = True
        # Two contributions: the head (loss) and the embedding. Autograd accumulates a leaf only after ALL
        # its backward edges have run, so if either contribution flows through autograd its accumulate hook
        # is the completion signal; only when both are written straight into the flat buffer does the
        # embedding backward (the last node of the graph) report the weight itself.
        head_direct = self.loss_impl == "sm100" or self.lm_head.impl != "torch"
        embed_direct = self.embed_impl == "sm100" or self.tp is not None
        w._manual_ready = head_direct and embed_direct
        for m in self.modules():
            if isinstance(m, Linear) and m.impl != "torch" and m.weight is not w:
                m.weight._manual_ready = True
            if isinstance(m, AddRMSNorm) and m.impl == "sm100":
                m.weight._manual_ready = True

    def reset_parameters(self):
        """N(0, init_std) for every matmul weight and the embedding; the two projections that write
        into the residual stream (wo, w_down) get init_std / sqrt(2 L) (GPT-2 scaled init)."""
        std = self.cfg.init_std
        nn.init.normal_(self.tok_emb.weight, std=std)
        resid_std = std / math.sqrt(2 * self.cfg.n_layers)
        for block in self.blocks:
            nn.init.normal_(block.attn.wqkv.weight, std=std)
            nn.init.normal_(block.mlp.w_gu.weight, std=std)
            nn.init.normal_(block.attn.wo.weight, std=resid_std)
            nn.init.normal_(block.mlp.w_down.weight, std=resid_std)
        for m in self.modules():
            if isinstance(m, AddRMSNorm):
                nn.init.ones_(m.weight)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None, loss_scale: float = 1.0):
        """idx, targets: (B, T) token ids. Returns (logits, loss). loss is None without targets;
        logits is None when targets are given and the fused linear+cross-entropy kernel is selected.
        `loss_scale` is only a hint for the fused loss (it lets it pre-scale its gradients)."""
        T = idx.shape[1]
        assert T <= self.cfg.max_seq_len, f"sequence length {T} > max_seq_len {self.cfg.max_seq_len}"
        if self.tp is not None:
            return self._forward_tp(idx, targets)
        x, delta = ops.embedding(idx, self.tok_emb.weight, impl=self.embed_impl), None
        for block in self.blocks:
            x, delta = block(x, self.rope_cos, self.rope_sin, delta)
        h = self.norm_out(x, delta)[0]
        if targets is not None and self.loss_impl == "sm100":
            loss = ops.linear_cross_entropy(h.reshape(-1, h.size(-1)), self.lm_head.weight, targets.reshape(-1))
            return None, loss
        logits = self.lm_head(h)
        loss = None
        if targets is not None:
            loss = F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))
        return logits, loss

    def _forward_tp(self, idx, targets):
        """Tensor + sequence parallel forward: token-sharded residual stream, vocabulary-sharded head."""
        from nanonemo_b200.parallel.tp import _VocabParallelCE, _VocabParallelEmbedding

        tp = self.tp
        tp.B, tp.T = idx.shape
        assert idx.numel() % tp.world == 0, "B * T must divide evenly over the tensor-parallel ranks"
        out_dtype = getattr(self, "residual_dtype", torch.float32) if self.embed_impl == "sm100" else self.tok_emb.weight.dtype
        x = _VocabParallelEmbedding.apply(idx.reshape(-1), self.tok_emb.weight, tp, self.vocab_start, out_dtype)
        delta = None
        for block in self.blocks:
            x, delta = block(x, self.rope_cos, self.rope_sin, delta)
        h = tp.gather_tokens(self.norm_out(x, delta)[0])
        if targets is not None and self.loss_impl == "sm100":
            from nanonemo_b200.ops.linear_ce import vocab_parallel_linear_cross_entropy

            return None, vocab_parallel_linear_cross_entropy(h, self.lm_head.weight, targets.reshape(-1), tp, self.vocab_start)
        logits = self.lm_head(h)  # [B*T, V / tp]
        if targets is None:
            return logits, None
        return logits, _VocabParallelCE.apply(logits, targets.reshape(-1), tp, self.vocab_start)

    def num_params(self, non_embedding: bool = False) -> int:
        n = sum(p.numel() for p in self.parameters())  # the tied weight is yielded once
        if non_embedding:
            n -= self.tok_emb.weight.numel()
        return n


if __name__ == "__main__":
    m = NanoNemo(ModelConfig())
    print(f"total params:         {m.num_params():,}")
    print(f"non-embedding params: {m.num_params(non_embedding=True):,}")
