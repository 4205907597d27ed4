"""LLaMA checkpoint interoperability (cf. fairseq2 ``models/llama/interop.py:20-214``):
key maps between this framework's names, Hugging Face ``LlamaForCausalLM`` and
Meta's reference implementation, including the rotary layout permutation (HF
stores q/k projections for half-rotation RoPE; this framework rotates
interleaved pairs)."""
from __future__ import annotations

import re
from typing import Any, Mapping

import torch
from torch import Tensor

from fairseq2_b200.models.llama.config import LLaMAConfig

_HG_KEY_MAP = {
    r"^model\.layers\.([0-9]+)\.self_attn\.q_proj\.": r"decoder.layers.\1.self_attn.q_proj.",
    r"^model\.layers\.([0-9]+)\.self_attn\.k_proj\.": r"decoder.layers.\1.self_attn.k_proj.",
    r"^model\.layers\.([0-9]+)\.self_attn\.v_proj\.": r"decoder.layers.\1.self_attn.v_proj.",
    r"^model\.layers\.([0-9]+)\.self_attn\.o_proj\.": r"decoder.layers.\1.self_attn.output_proj.",
    r"^model\.layers\.([0-9]+)\.post_attention_layernorm\.": r"decoder.layers.\1.ffn_layer_norm.",
    r"^model\.layers\.([0-9]+)\.mlp\.gate_proj\.": r"decoder.layers.\1.ffn.gate_proj.",
    r"^model\.layers\.([0-9]+)\.mlp\.down_proj\.": r"decoder.layers.\1.ffn.output_proj.",
    r"^model\.layers\.([0-9]+)\.mlp\.up_proj\.": r"decoder.layers.\1.ffn.inner_proj.",
    r"^model\.layers\.([0-9]+)\.input_layernorm\.": r"decoder.layers.\1.self_attn_layer_norm.",
    r"^model\.norm\.": r"decoder.layer_norm.",
    r"^model\.embed_tokens\.": r"decoder_frontend.embed.",
    r"^lm_head\.": r"final_proj.",
}

_REFERENCE_KEY_MAP = {
    r"^layers\.([0-9]+)\.attention\.wq\.": r"decoder.layers.\1.self_attn.q_proj.",
    r"^layers\.([0-9]+)\.attention\.wk\.": r"decoder.layers.\1.self_attn.k_proj.",
    r"^layers\.([0-9]+)\.attention\.wv\.": r"decoder.layers.\1.self_attn.v_proj.",
    r"^layers\.([0-9]+)\.attention\.wo\.": r"decoder.layers.\1.self_attn.output_proj.",
    r"^layers\.([0-9]+)\.attention_norm\.": r"decoder.layers.\1.self_attn_layer_norm.",
    r"^layers\.([0-9]+)\.feed_forward\.w1\.": r"decoder.layers.\1.ffn.gate_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.w2\.": r"decoder.layers.\1.ffn.output_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.w3\.": r"decoder.layers.\1.ffn.inner_proj.",
    r"^layers\.([0-9]+)\.ffn_norm\.": r"decoder.layers.\1.ffn_layer_norm.",
    r"^norm\.": r"decoder.layer_norm.",
    r"^tok_embeddings\.": r"decoder_frontend.embed.",
    r"^output\.": r"final_proj.",
}


def convert_state_dict(sd: Mapping[str, Any], key_map: Mapping[str, str]) -> dict[str, Any]:
    pats = [(re.compile(p), r) for p, r in key_map.items()]
    out: dict[str, Any] = {}
    for k, v in sd.items():
        nk = k
        for p, r in pats:
            nk, n = p.subn(r, k)
            if n:
                break
        out[nk] = v
    return out


def _hf_to_interleaved(w: Tensor, num_heads: int) -> Tensor:
    """HF layout: per head rows are [first halves | second halves]; interleave them."""
    d0, d1 = w.shape
    hd = d0 // num_heads
    return w.view(num_heads, 2, hd // 2, d1).transpose(1, 2).reshape(d0, d1)


def _interleaved_to_hf(w: Tensor, num_heads: int) -> Tensor:
    d0, d1 = w.shape
    hd = d0 // num_heads
    return w.view(num_heads, hd // 2, 2, d1).transpose(1, 2).reshape(d0, d1)


def convert_llama_state_dict(sd: dict[str, Any], config: LLaMAConfig) -> dict[str, Any]:
    """Accepts HF, Meta-reference or native keys and returns native keys/layout."""
    if any(k.startswith("model.layers.") or k.startswith("model.embed_tokens") for k in sd):
        out = convert_state_dict(sd, _HG_KEY_MAP)
        for k in list(out):
            if k.endswith("self_attn.q_proj.weight"):
                out[k] = _hf_to_interleaved(out[k], config.num_attn_heads)
            elif k.endswith("self_attn.k_proj.weight"):
                out[k] = _hf_to_interleaved(out[k], config.num_key_value_heads)
        if config.tied_embeddings:
            out.pop("final_proj.weight", None)
        out = {k: v for k, v in out.items() if not k.endswith("rotary_emb.inv_freq")}
        return out
    if any(k.startswith("layers.") or k.startswith("tok_embeddings.") for k in sd):
        out = convert_state_dict(sd, _REFERENCE_KEY_MAP)
        out.pop("rope.freqs", None)
        if config.tied_embeddings:
            out.pop("final_proj.weight", None)
        return out
    return dict(sd)


def export_llama_to_hg(sd: Mapping[str, Any], config: LLaMAConfig) -> tuple[dict[str, Any], dict[str, Any]]:
    """Native consolidated state dict -> (HF state dict, HF ``config.json`` dict)."""
    inv = {}
    for p, r in _HG_KEY_MAP.items():
        src = r.replace("\\1", "([0-9]+)").replace(".", r"\.")
        dst = p.strip("^").replace("([0-9]+)", r"\1").replace("\\.", ".")
        inv["^" + src] = dst
    out = convert_state_dict(sd, inv)
    for k in list(out):
        if k.endswith("self_attn.q_proj.weight"):
            out[k] = _interleaved_to_hf(out[k], config.num_attn_heads)
        elif k.endswith("self_attn.k_proj.weight"):
            out[k] = _interleaved_to_hf(out[k], config.num_key_value_heads)
    if config.tied_embeddings and "lm_head.weight" not in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    multiple = config.ffn_inner_dim_multiple_of
    inner = int(config.ffn_inner_dim * config.ffn_inner_dim_multiplier * config.ffn_inner_dim_scale)
    inner = multiple * ((inner + multiple - 1) // multiple)
    hf_config = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": config.model_dim,
        "intermediate_size": inner, "num_hidden_layers": config.num_layers,
        "num_attention_heads": config.num_attn_heads, "num_key_value_heads": config.num_key_value_heads,
        "vocab_size": config.vocab_size, "max_position_embeddings": config.max_seq_len,
        "rope_theta": config.rope_theta, "rms_norm_eps": 1e-5, "tie_word_embeddings": config.tied_embeddings,
        "hidden_act": "silu", "torch_dtype": "bfloat16",
    }
    if config.use_scaled_rope:
        hf_config["rope_scaling"] = {"rope_type": "llama3", "factor": config.rope_scale.factor,
                                     "low_freq_factor": config.rope_scale.frequency_factors[0],
                                     "high_freq_factor": config.rope_scale.frequency_factors[1],
                                     "original_max_position_embeddings": config.rope_scale.original_context_length}
    return out, hf_config
