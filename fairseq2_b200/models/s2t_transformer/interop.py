"""Conversion of original fairseq S2T checkpoints (cf. fairseq2 ``models/s2t_transformer/interop.py:17-52``,
``models/s2t_conformer/interop.py``)."""
from __future__ import annotations

from typing import Any

from fairseq2_b200.models.utils_fairseq import FAIRSEQ_ENC_DEC_KEY_MAP, convert_fairseq_state_dict

_S2T = dict(FAIRSEQ_ENC_DEC_KEY_MAP)
_S2T.update({
    r"^encoder\.subsample\.conv_layers\.([0-9]+)\.": r"encoder_frontend.feature_extractor.layers.\1.conv.",
    r"^encoder\.transformer_layers\.([0-9]+)\.self_attn\.out_proj\.": r"encoder.layers.\1.self_attn.output_proj.",
    r"^encoder\.transformer_layers\.([0-9]+)\.fc1\.": r"encoder.layers.\1.ffn.inner_proj.",
    r"^encoder\.transformer_layers\.([0-9]+)\.fc2\.": r"encoder.layers.\1.ffn.output_proj.",
    r"^encoder\.transformer_layers\.([0-9]+)\.final_layer_norm\.": r"encoder.layers.\1.ffn_layer_norm.",
    r"^encoder\.transformer_layers\.([0-9]+)\.": r"encoder.layers.\1.",
    r"^encoder\.linear\.": r"encoder_frontend.proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.ffn(1|2)\.layer_norm\.": r"encoder.layers.\1.ffn\2_layer_norm.",
    r"^encoder\.conformer_layers\.([0-9]+)\.ffn(1|2)\.w_1\.": r"encoder.layers.\1.ffn\2.inner_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.ffn(1|2)\.w_2\.": r"encoder.layers.\1.ffn\2.output_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn_layer_norm\.": r"encoder.layers.\1.self_attn_layer_norm.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.linear_q\.": r"encoder.layers.\1.self_attn.q_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.linear_k\.": r"encoder.layers.\1.self_attn.k_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.linear_v\.": r"encoder.layers.\1.self_attn.v_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.linear_out\.": r"encoder.layers.\1.self_attn.output_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.linear_pos\.": r"encoder.layers.\1.self_attn.sdpa.r_proj.",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.pos_bias_u$": r"encoder.layers.\1.self_attn.sdpa.u_bias",
    r"^encoder\.conformer_layers\.([0-9]+)\.self_attn\.pos_bias_v$": r"encoder.layers.\1.self_attn.sdpa.v_bias",
    r"^encoder\.conformer_layers\.([0-9]+)\.conv_module\.layer_norm\.": r"encoder.layers.\1.conv_layer_norm.",
    r"^encoder\.conformer_layers\.([0-9]+)\.conv_module\.": r"encoder.layers.\1.conv.",
    r"^encoder\.conformer_layers\.([0-9]+)\.final_layer_norm\.": r"encoder.layers.\1.layer_norm.",
})


def convert_s2t_state_dict(sd: dict[str, Any], config: Any) -> dict[str, Any]:
    inner = sd.get("model", sd)
    if "decoder.embed_tokens.weight" not in inner:
        return {k.removeprefix("module."): v for k, v in inner.items()}
    return convert_fairseq_state_dict(sd, _S2T)
