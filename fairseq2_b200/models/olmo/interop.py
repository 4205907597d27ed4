"""OLMo checkpoint conversion (cf. fairseq2 ``models/olmo/interop.py``): Hugging Face
``Olmo2ForCausalLM`` / ``Olmo3ForCausalLM``. HF names the post-sub-layer norms
``post_attention_layernorm`` and ``post_feedforward_layernorm``."""
from __future__ import annotations

from typing import Any, Mapping

from fairseq2_b200.models.olmo.config import OLMOConfig
from fairseq2_b200.models.utils_hg_lm import HG_LM_KEY_MAP, convert_hg_lm_state_dict, export_hg_lm_state_dict

_OLMO_KEY_MAP = {k: v for k, v in HG_LM_KEY_MAP.items() if "layernorm" not in k}
_OLMO_KEY_MAP.update({
    r"^model\.layers\.([0-9]+)\.post_attention_layernorm\.": r"decoder.layers.\1.self_attn_layer_norm.",
    r"^model\.layers\.([0-9]+)\.post_feedforward_layernorm\.": r"decoder.layers.\1.ffn_layer_norm.",
})


def convert_olmo_state_dict(sd: dict[str, Any], config: OLMOConfig) -> dict[str, Any]:
    return convert_hg_lm_state_dict(sd, num_heads=config.num_attn_heads, num_kv_heads=config.num_key_value_heads,
                                    tied=config.tied_embeddings, per_head_norm=False, key_map=_OLMO_KEY_MAP)


def export_olmo_to_hg(sd: Mapping[str, Any], config: OLMOConfig) -> tuple[dict[str, Any], dict[str, Any]]:
    out = export_hg_lm_state_dict(sd, num_heads=config.num_attn_heads, num_kv_heads=config.num_key_value_heads,
                                  tied=config.tied_embeddings, per_head_norm=False, key_map=_OLMO_KEY_MAP)
    v3 = config.sliding_window is not None
    hf: dict[str, Any] = {
        "architectures": ["Olmo3ForCausalLM" if v3 else "Olmo2ForCausalLM"], "model_type": "olmo3" if v3 else "olmo2",
        "hidden_size": config.model_dim, "intermediate_size": config.ffn_inner_dim,
        "num_hidden_layers": config.num_layers, "num_attention_heads": config.num_attn_heads,
        "num_key_value_heads": config.num_key_value_heads, "vocab_size": config.vocab_size,
        "max_position_embeddings": config.max_seq_len, "rope_theta": config.rope_theta,
        "rms_norm_eps": config.rms_norm_eps, "hidden_act": "silu", "tie_word_embeddings": config.tied_embeddings,
        "pad_token_id": config.pad_idx, "eos_token_id": config.eos_token_id, "torch_dtype": "bfloat16"}
    if v3:
        hf["sliding_window"] = config.sliding_window
        hf["layer_types"] = config.resolved_layer_types()
    if config.yarn_scale_config is not None:
        y = config.yarn_scale_config
        hf["rope_scaling"] = {"rope_type": "yarn", "factor": y.scale_factor,
                              "original_max_position_embeddings": y.original_max_seq_len, "beta_fast": y.beta_fast,
                              "beta_slow": y.beta_slow, "attention_factor": None}
    return out, hf
