"""LLaMA-4 checkpoint conversion (cf. fairseq2 ``models/llama4/interop.py:20-149``): the original
release format with merged ``wqkv`` matrices, fused norm weights and stacked expert tensors."""
from __future__ import annotations

import re
from typing import Any

from fairseq2_b200.models.llama.interop import convert_state_dict
from fairseq2_b200.models.llama4.config import Llama4Config

_KEY_MAP = {
    r"^layers\.([0-9]+)\.attention\.wq\.": r"decoder.layers.\1.self_attn.q_proj.",
    r"^layers\.([0-9]+)\.attention\.wk\.": r"decoder.layers.\1.self_attn.k_proj.",
    r"^layers\.([0-9]+)\.attention\.wv\.": r"decoder.layers.\1.self_attn.v_proj.",
    r"^layers\.([0-9]+)\.attention\.wo\.": r"decoder.layers.\1.self_attn.output_proj.",
    r"^layers\.([0-9]+)\.attention\.wqkv\.layer_norm_weight$": r"decoder.layers.\1.self_attn_layer_norm.weight",
    r"^layers\.([0-9]+)\.attention_norm\.": r"decoder.layers.\1.self_attn_layer_norm.",
    r"^layers\.([0-9]+)\.feed_forward\.w1\.": r"decoder.layers.\1.ffn.gate_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.w2\.": r"decoder.layers.\1.ffn.output_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.mlp\.fc2_weight$": r"decoder.layers.\1.ffn.output_proj.weight",
    r"^layers\.([0-9]+)\.feed_forward\.w3\.": r"decoder.layers.\1.ffn.inner_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.mlp\.layer_norm_weight$": r"decoder.layers.\1.ffn_layer_norm.weight",
    r"^layers\.([0-9]+)\.feed_forward\.router_DE$": r"decoder.layers.\1.ffn.router",
    r"^layers\.([0-9]+)\.feed_forward\.norm\.": r"decoder.layers.\1.ffn_layer_norm.",
    r"^layers\.([0-9]+)\.ffn_norm\.": r"decoder.layers.\1.ffn_layer_norm.",
    r"^layers\.([0-9]+)\.feed_forward\.w_in_shared_FD\.": r"decoder.layers.\1.ffn.shared_expert.gate_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.w_swiglu_FD\.": r"decoder.layers.\1.ffn.shared_expert.inner_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.w_out_shared_DF\.": r"decoder.layers.\1.ffn.shared_expert.output_proj.",
    r"^layers\.([0-9]+)\.feed_forward\.experts\.moe_w_in_eD_F$": r"decoder.layers.\1.ffn.experts.gate_proj",
    r"^layers\.([0-9]+)\.feed_forward\.experts\.moe_w_swiglu_eD_F$": r"decoder.layers.\1.ffn.experts.inner_proj",
    r"^layers\.([0-9]+)\.feed_forward\.experts\.moe_w_out_eF_D$": r"decoder.layers.\1.ffn.experts.output_proj",
    r"^norm\.": r"decoder.layer_norm.",
    r"^tok_embeddings\.": r"decoder_frontend.embed.",
    r"^output\.": r"final_proj.",
}

_SKIP = ("rope.freqs", "._extra_state", ".expert_activation_DE", "_stats_3E")


def convert_llama4_state_dict(sd: dict[str, Any], config: Llama4Config) -> dict[str, Any]:
    if not any(k.startswith("layers.") or k.startswith("tok_embeddings.") for k in sd):
        return dict(sd)
    hd = config.model_dim // config.num_attn_heads
    src: dict[str, Any] = {}
    for k, v in sd.items():
        if any(s in k for s in _SKIP) or k.startswith("vision_") or k.startswith("speech_"):
            continue
        if re.match(r"layers\.[0-9]+\.attention\.wqkv\.weight$", k):
            # a (possibly tensor-parallel) shard of the merged projection: q rows, then k rows, then v rows
            full = (config.num_attn_heads + 2 * config.num_key_value_heads) * hd
            tp = max(full // v.shape[0], 1)
            nq = config.num_attn_heads // tp * hd
            nkv = max(1, config.num_key_value_heads // tp) * hd
            src[k.replace(".wqkv.", ".wq.")] = v[:nq]
            src[k.replace(".wqkv.", ".wk.")] = v[nq:nq + nkv]
            src[k.replace(".wqkv.", ".wv.")] = v[nq + nkv:nq + 2 * nkv]
        else:
            src[k] = v
    out = convert_state_dict(src, _KEY_MAP)
    E = config.experts.num_experts
    for k in list(out):
        if ".ffn.experts." in k and out[k].ndim == 2:
            # stacked experts are stored flattened as [(E·rows), cols]
            out[k] = out[k].view(E, out[k].shape[0] // E, out[k].shape[1])
    return out
