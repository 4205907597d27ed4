"""Hugging Face <-> fairseq2_b200 state dicts for Gemma 3n (text decoder). Module names follow the Hugging Face
layout, so conversion is a prefix change: ``model.`` (``Gemma3nForCausalLM``) or ``model.language_model.``
(``Gemma3nForConditionalGeneration``) is dropped; audio tower entries are kept when the config has an audio
tower, vision entries are skipped
(cf. fairseq2 ``models/gemma3n/interop.py:30-267``)."""
from __future__ import annotations

from typing import Any

from torch import Tensor

from fairseq2_b200.models.gemma3n.config import Gemma3nConfig

_VISION = ("model.vision_tower.", "model.embed_vision.")
_AUDIO = ("model.audio_tower.", "model.embed_audio.")


def convert_gemma3n_state_dict(state_dict: dict[str, Tensor], config: Gemma3nConfig) -> dict[str, Tensor]:
    if not any(k.startswith("model.") for k in state_dict):
        return state_dict                                        # already in the native layout
    out: dict[str, Tensor] = {}
    for key, value in state_dict.items():
        if key.startswith(_VISION) or (config.audio_config is None and key.startswith(_AUDIO)):
            continue
        if key.startswith(_AUDIO):
            if not key.endswith("embedding_post_projection_norm.weight"):
                out[key[len("model."):]] = value
            continue
        if key.startswith("model.language_model."):
            key = key[len("model.language_model."):]
        elif key.startswith("model."):
            key = key[len("model."):]
        elif key == "lm_head.weight":
            if config.tied_embeddings:
                continue
        out[key] = value
    return out


def export_gemma3n_to_hg(state_dict: dict[str, Tensor], config: Gemma3nConfig) -> tuple[dict[str, Tensor], dict[str, Any]]:
    """Returns ``(Gemma3nForCausalLM state dict, text config dict)``."""
    sd = {("lm_head.weight" if k == "lm_head.weight" else "model." + k): v for k, v in state_dict.items()}
    L = config.num_layers
    from fairseq2_b200.models.gemma3n.config import is_global_layer

    hg = {
        "architectures": ["Gemma3nForCausalLM"], "model_type": "gemma3n_text", "vocab_size": config.vocab_size,
        "vocab_size_per_layer_input": config.vocab_size_per_layer_input, "hidden_size": config.model_dim,
        "hidden_size_per_layer_input": config.hidden_size_per_layer_input,
        "intermediate_size": [config.ffn_inner_dim] * L, "num_hidden_layers": L,
        "num_attention_heads": config.num_attn_heads, "num_key_value_heads": config.num_key_value_heads,
        "head_dim": config.head_dim, "max_position_embeddings": config.max_seq_len,
        "sliding_window": config.sliding_window, "rms_norm_eps": config.rms_norm_eps,
        "layer_types": ["full_attention" if is_global_layer(i, L) else "sliding_attention" for i in range(L)],
        "rope_theta": config.rope_theta_global, "rope_local_base_freq": config.rope_theta,
        "final_logit_softcapping": config.final_logit_soft_cap, "num_kv_shared_layers": config.num_kv_shared_layers,
        "laurel_rank": config.laurel_rank, "altup_num_inputs": config.altup_num_inputs,
        "altup_active_idx": config.altup_active_idx, "altup_coef_clip": config.altup_coef_clip,
        "altup_correct_scale": config.altup_correct_scale,
        "activation_sparsity_pattern": [config.activation_sparsity if i < config.num_sparse_layers else 0.0 for i in range(L)],
        "hidden_activation": "gelu_pytorch_tanh", "pad_token_id": config.pad_idx,
        "tie_word_embeddings": config.tied_embeddings,
    }
    return sd, hg
