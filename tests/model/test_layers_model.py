"""Model blocks against independently written references; model-level invariants (CPU)."""

import math

import pytest
import torch
import torch.nn.functional as F

from nanonemo_b200 import ops
from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.layers import MLP, AddRMSNorm, Attention, Block, RMSNorm, apply_rope, rope_cache
from nanonemo_b200.models.model import NanoNemo

SMALL = dict(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=32)


def test_rmsnorm_formula_and_torch_builtin():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 16)
    norm = RMSNorm(16, eps=1e-5)
    norm.weight.data = torch.rand(16) + 0.5
    by_hand = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * norm.weight
    torch.testing.assert_close(norm(x), by_hand)
    torch.testing.assert_close(norm(x), F.rms_norm(x, (16,), norm.weight, 1e-5))


def test_add_rms_norm_returns_sum_and_handles_no_delta():
    n = AddRMSNorm(8)
    x, d = torch.randn(2, 3, 8), torch.randn(2, 3, 8)
    y, h = n(x, d)
    torch.testing.assert_close(h, x + d)
    torch.testing.assert_close(y, RMSNorm.forward(n, x + d))
    y0, h0 = n(x)
    assert h0 is x
    torch.testing.assert_close(y0, RMSNorm.forward(n, x))


def test_rope_matches_complex_rotation_and_is_relative():
    torch.manual_seed(1)
    hd, T = 16, 12
    cos, sin = rope_cache(hd, 32)
    x = torch.randn(1, 2, T, hd)
    out = apply_rope(x, cos, sin)
    # complex form: pair (i, i + hd/2) rotates by angle m * theta_i
    theta = 10000.0 ** (-torch.arange(0, hd, 2).float() / hd)
    ang = torch.outer(torch.arange(T).float(), theta)
    z = torch.complex(x[..., : hd // 2], x[..., hd // 2:]) * torch.polar(torch.ones_like(ang), ang)
    torch.testing.assert_close(out, torch.cat((z.real, z.imag), -1), rtol=1e-5, atol=1e-5)
    # relative-position property: <R_m q, R_n k> depends on m - n only
    q, k = torch.randn(hd), torch.randn(hd)
    def rot(v, m):
        return apply_rope(v.view(1, 1, 1, hd).expand(1, 1, m + 1, hd).contiguous(), cos, sin)[0, 0, m]
    torch.testing.assert_close(rot(q, 5) @ rot(k, 2), rot(q, 9) @ rot(k, 6), rtol=1e-4, atol=1e-4)
    assert torch.allclose(out[:, :, 0], x[:, :, 0])  # position 0 is not rotated


def reference_attention(attn: Attention, x, cos, sin):
    """Explicit per-head loop; query head h uses KV head h // group."""
    B, T, _ = x.shape
    wq, wk, wv = attn.split_qkv()
    H, KVH, hd = attn.n_heads, attn.n_kv_heads, attn.head_dim
    q = (x @ wq.t()).view(B, T, H, hd).transpose(1, 2)
    k = (x @ wk.t()).view(B, T, KVH, hd).transpose(1, 2)
    v = (x @ wv.t()).view(B, T, KVH, hd).transpose(1, 2)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = torch.zeros(B, T, H * hd)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // KVH)
        s = (q[:, h] @ k[:, g].transpose(-1, -2)) / math.sqrt(hd)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, :, h * hd:(h + 1) * hd] = torch.softmax(s, -1) @ v[:, g]
    return out @ attn.wo.weight.t()


@pytest.mark.parametrize("backend", ["math", "mem_efficient"])
def test_attention_matches_per_head_loop_and_is_causal(backend):
    torch.manual_seed(2)
    cfg = ModelConfig(**SMALL, attn_backend="math")
    attn = Attention(cfg)
    for w in (attn.wqkv.weight, attn.wo.weight):
        torch.nn.init.normal_(w, std=0.1)
    cos, sin = rope_cache(cfg.head_dim, 32)
    x = torch.randn(2, 10, 64)
    out = attn(x, cos, sin)
    torch.testing.assert_close(out, reference_attention(attn, x, cos, sin), rtol=1e-4, atol=1e-5)
    x2 = x.clone()
    x2[:, 6:] += 1.0  # perturb the future
    torch.testing.assert_close(attn(x2, cos, sin)[:, :6], out[:, :6])


def test_packed_ops_match_unpacked():
    torch.manual_seed(3)
    B, T, H, KVH, hd = 2, 8, 4, 2, 16
    cos, sin = rope_cache(hd, 16)
    qkv = torch.randn(B, T, (H + 2 * KVH) * hd)
    rot = ops.rope_qkv(qkv, cos, sin, H, KVH, hd)
    q, k, v = qkv.split((H * hd, KVH * hd, KVH * hd), -1)
    q_ref = apply_rope(q.view(B, T, H, hd).transpose(1, 2), cos, sin)
    torch.testing.assert_close(rot[..., : H * hd].view(B, T, H, hd).transpose(1, 2), q_ref)
    torch.testing.assert_close(rot[..., (H + KVH) * hd:], v)
    out = ops.attention_packed(rot, H, KVH, hd)
    k_ref = apply_rope(k.view(B, T, KVH, hd).transpose(1, 2), cos, sin)
    ref = ops.attention_torch(q_ref, k_ref, v.view(B, T, KVH, hd).transpose(1, 2))
    torch.testing.assert_close(out, ref.transpose(1, 2).reshape(B, T, -1))


def test_mlp_identities():
    cfg = ModelConfig(**SMALL)
    mlp = MLP(cfg)
    torch.nn.init.normal_(mlp.w_gu.weight, std=0.1)
    torch.nn.init.normal_(mlp.w_down.weight, std=0.1)
    x = torch.randn(3, 64)
    g, u = mlp.split_gu()
    torch.testing.assert_close(mlp(x), (F.silu(x @ g.t()) * (x @ u.t())) @ mlp.w_down.weight.t())
    mlp.w_gu.weight.data[: cfg.d_ff] = 0  # closed gate: silu(0) = 0
    assert mlp(x).abs().max() == 0


def test_block_residual_stream_convention():
    torch.manual_seed(4)
    cfg = ModelConfig(**SMALL)
    blk = Block(cfg)
    cos, sin = rope_cache(cfg.head_dim, 32)
    x, d = torch.randn(1, 6, 64), torch.randn(1, 6, 64)
    x1, m = blk(x, cos, sin, d)
    h = x + d
    a = blk.attn(RMSNorm.forward(blk.norm_attn, h), cos, sin)
    torch.testing.assert_close(x1, h + a)
    torch.testing.assert_close(m, blk.mlp(RMSNorm.forward(blk.norm_mlp, h + a)))
    blk.attn.wo.weight.data.zero_()
    blk.mlp.w_down.weight.data.zero_()
    x2, m2 = blk(x, cos, sin, d)
    torch.testing.assert_close(x2, h)
    assert m2.abs().max() == 0


def test_param_count_tying_buffers_and_init():
    m = NanoNemo(ModelConfig())
    assert m.num_params() == 114_150_144 and m.num_params(non_embedding=True) == 75_516_672
    assert m.lm_head.weight is m.tok_emb.weight
    assert not any("rope" in k for k in m.state_dict())
    assert len([n for n, _ in m.named_parameters()]) == 1 + 12 * 6 + 1
    std = m.blocks[0].attn.wqkv.weight.std().item()
    resid = m.blocks[0].attn.wo.weight.std().item()
    assert abs(std - 0.02) < 2e-3 and abs(resid - 0.02 / math.sqrt(24)) < 5e-4
    assert abs(m.blocks[3].mlp.w_down.weight.std().item() - 0.02 / math.sqrt(24)) < 5e-4


def test_initial_loss_is_log_vocab():
    torch.manual_seed(0)
    cfg = ModelConfig(n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, d_ff=256, vocab_size=50304, max_seq_len=64)
    m = NanoNemo(cfg)
    idx = torch.randint(0, 50257, (4, 65))
    _, loss = m(idx[:, :-1], idx[:, 1:])
    assert abs(loss.item() - math.log(50304)) < 0.1
    logits, none = m(idx[:, :-1])
    assert none is None and logits.shape == (4, 64, 50304)
    with pytest.raises(AssertionError):
        m(torch.zeros(1, 65, dtype=torch.long))


def test_config_validation_and_aliases():
    with pytest.raises(AssertionError):
        ModelConfig(n_heads=12, n_kv_heads=5)
    with pytest.raises(AssertionError):
        ModelConfig(norm_kernel="fast")
    r = ModelConfig(norm_kernel="cuda", swiglu_kernel="triton", loss_kernel="fused", linear_impl="te").resolved()
    assert (r.norm_kernel, r.swiglu_kernel, r.loss_kernel, r.linear_impl, r.rope_kernel) == ("sm100", "sm100", "sm100", "mxfp8", "torch")
    assert ModelConfig(n_layers=24, d_model=2048, n_heads=16, n_kv_heads=4, d_ff=5632).head_dim == 128


def test_sm100_ops_refuse_cpu_tensors():
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.add_rms_norm(torch.randn(2, 8), None, torch.ones(8), 1e-5, impl="sm100")


def test_overfits_one_batch():
    torch.manual_seed(0)
    m = NanoNemo(ModelConfig(**SMALL))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    idx = torch.randint(0, 512, (4, 17))
    first = None
    for _ in range(60):
        _, loss = m(idx[:, :-1], idx[:, 1:])
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.3 * first
