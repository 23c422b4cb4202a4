"""Export to the Hugging Face Llama format (safetensors), for lm-eval's ``hf`` backend or any HF tool.

The architecture maps one-to-one onto ``LlamaForCausalLM`` (pre-norm RMSNorm eps 1e-5, rotate-half
RoPE base 10000, SwiGLU, GQA with query head h on KV head h // group, no biases, tied embeddings),
as in the reference exporter (nanonemo/eval/hf_export.py:22-83). This framework stores the Q/K/V
projections and the gate/up projections as single fused parameters; the exporter splits them back
into q/k/v_proj and gate/up_proj. ``load_checkpoint`` reads only the model part of a training
checkpoint, whatever layout wrote it (they all store the same per-projection names).
"""

import pathlib
import sys
from pathlib import Path

import torch

from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.model import NanoNemo

EOT = 50256


def llama_config(cfg: ModelConfig):
    from transformers import LlamaConfig

    return LlamaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.d_model, intermediate_size=cfg.d_ff,
                       num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.n_heads,
                       num_key_value_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                       max_position_embeddings=cfg.max_seq_len, rms_norm_eps=cfg.norm_eps, rope_theta=cfg.rope_base,
                       hidden_act="silu", attention_bias=False, mlp_bias=False, tie_word_embeddings=True,
                       bos_token_id=EOT, eos_token_id=EOT, torch_dtype="float32")


def hf_state_dict(model: NanoNemo) -> dict[str, torch.Tensor]:
    out = {"model.embed_tokens.weight": model.tok_emb.weight, "model.norm.weight": model.norm_out.weight,
           "lm_head.weight": model.lm_head.weight}
    for i, block in enumerate(model.blocks):
        pre = f"model.layers.{i}."
        q, k, v = block.attn.split_qkv()
        gate, up = block.mlp.split_gu()
        out.update({pre + "input_layernorm.weight": block.norm_attn.weight, pre + "self_attn.q_proj.weight": q,
                    pre + "self_attn.k_proj.weight": k, pre + "self_attn.v_proj.weight": v,
                    pre + "self_attn.o_proj.weight": block.attn.wo.weight,
                    pre + "post_attention_layernorm.weight": block.norm_mlp.weight,
                    pre + "mlp.gate_proj.weight": gate, pre + "mlp.up_proj.weight": up,
                    pre + "mlp.down_proj.weight": block.mlp.w_down.weight})
    return {name: t.detach().float().cpu().contiguous() for name, t in out.items()}


def to_hf(model: NanoNemo):
    from transformers import LlamaForCausalLM

    hf = LlamaForCausalLM(llama_config(model.cfg))
    hf.load_state_dict(hf_state_dict(model), strict=True)
    return hf.eval()


def load_checkpoint(path, cfg: ModelConfig) -> NanoNemo:
    """Weights of a training checkpoint (the optimizer part is not read) into a CPU model. Works for checkpoints of this
    framework and of the reference alike: both store the per-projection names (train/checkpoint.py)."""
    from nanonemo_b200.train.checkpoint import restore_state

    sys.modules.setdefault("pathlib._local", pathlib)  # checkpoints pickled under Python 3.13 name this module
    model = NanoNemo(cfg)
    restore_state(path, model, None, device="cpu")
    return model.eval()


def export(model: NanoNemo, out_dir, tokenizer: bool = True) -> Path:
    out_dir = Path(out_dir)
    to_hf(model).save_pretrained(out_dir, safe_serialization=True)
    if tokenizer:
        from transformers import AutoTokenizer

        AutoTokenizer.from_pretrained("gpt2").save_pretrained(out_dir)  # needs a cached or downloadable GPT-2 tokenizer
    return out_dir
