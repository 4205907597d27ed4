"""Qwen checkpoint conversion (cf. fairseq2 ``models/qwen/interop.py``): Hugging Face
``Qwen2ForCausalLM`` / ``Qwen3ForCausalLM``."""
from __future__ import annotations

from typing import Any, Mapping

from fairseq2_b200.models.qwen.config import QwenConfig
from fairseq2_b200.models.utils_hg_lm import convert_hg_lm_state_dict, export_hg_lm_state_dict


def convert_qwen_state_dict(sd: dict[str, Any], config: QwenConfig) -> dict[str, Any]:
    return convert_hg_lm_state_dict(sd, num_heads=config.num_attn_heads, num_kv_heads=config.num_key_value_heads,
                                    tied=config.tied_embeddings, per_head_norm=True)


def export_qwen_to_hg(sd: Mapping[str, Any], config: QwenConfig) -> tuple[dict[str, Any], dict[str, Any]]:
    out = export_hg_lm_state_dict(sd, num_heads=config.num_attn_heads, num_kv_heads=config.num_key_value_heads,
                                  tied=config.tied_embeddings, per_head_norm=True)
    v3 = config.q_norm or config.k_norm
    hd = config.head_dim if config.head_dim is not None else config.model_dim // config.num_attn_heads
    hf = {"architectures": ["Qwen3ForCausalLM" if v3 else "Qwen2ForCausalLM"], "model_type": "qwen3" if v3 else "qwen2",
          "hidden_size": config.model_dim, "intermediate_size": config.ffn_inner_dim,
          "num_hidden_layers": config.num_layers, "num_attention_heads": config.num_attn_heads,
          "num_key_value_heads": config.num_key_value_heads, "head_dim": hd, "vocab_size": config.vocab_size,
          "max_position_embeddings": config.max_seq_len, "rope_theta": config.rope_theta, "rms_norm_eps": 1e-6,
          "hidden_act": "silu", "tie_word_embeddings": config.tied_embeddings, "attention_bias": config.qkv_proj_bias,
          "torch_dtype": "bfloat16"}
    return out, hf
