"""Mistral checkpoint conversion (cf. fairseq2 ``models/mistral/interop.py``): Hugging Face
``MistralForCausalLM`` and the original ``consolidated`` format."""
from __future__ import annotations

from typing import Any, Mapping

from fairseq2_b200.models.llama.interop import _REFERENCE_KEY_MAP, convert_state_dict
from fairseq2_b200.models.mistral.config import MistralConfig
from fairseq2_b200.models.utils_hg_lm import convert_hg_lm_state_dict, export_hg_lm_state_dict, is_hg_state_dict


def convert_mistral_state_dict(sd: dict[str, Any], config: MistralConfig) -> dict[str, Any]:
    if is_hg_state_dict(sd):
        return convert_hg_lm_state_dict(sd, num_heads=config.num_attn_heads, num_kv_heads=config.num_key_value_heads,
                                        tied=False)
    if any(k.startswith("layers.") or k.startswith("tok_embeddings.") for k in sd):
        # the original release uses the Meta key names and already rotates interleaved pairs
        return convert_state_dict(sd, _REFERENCE_KEY_MAP)
    return dict(sd)


def export_mistral_to_hg(sd: Mapping[str, Any], config: MistralConfig) -> tuple[dict[str, Any], dict[str, Any]]:
    out = export_hg_lm_state_dict(sd, num_heads=config.num_attn_heads, num_kv_heads=config.num_key_value_heads,
                                  tied=False)
    hf = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_size": config.model_dim,
          "intermediate_size": config.ffn_inner_dim, "num_hidden_layers": config.num_layers,
          "num_attention_heads": config.num_attn_heads, "num_key_value_heads": config.num_key_value_heads,
          "vocab_size": config.vocab_size, "max_position_embeddings": config.max_seq_len,
          "sliding_window": config.attn_window_len, "rope_theta": config.rope_theta, "rms_norm_eps": 1e-5,
          "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16"}
    return out, hf
