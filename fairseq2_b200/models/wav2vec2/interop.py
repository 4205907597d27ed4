"""Conversion of original fairseq wav2vec 2.0 checkpoints (cf. fairseq2 ``models/wav2vec2/interop.py:19-64``,
``models/wav2vec2/asr/interop.py``) and of Hugging Face ``Wav2Vec2ForCTC`` state dicts."""
from __future__ import annotations

from typing import Any

import torch

from fairseq2_b200.models.llama.interop import convert_state_dict
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder

_COMMON = {
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layers\.([0-9]+)\.self_attn\.out_proj\.": r"encoder.layers.\2.self_attn.output_proj.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layers\.([0-9]+)\.self_attn\.(q|k|v)_proj\.": r"encoder.layers.\2.self_attn.\3_proj.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layers\.([0-9]+)\.self_attn_layer_norm\.": r"encoder.layers.\2.self_attn_layer_norm.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layers\.([0-9]+)\.fc1\.": r"encoder.layers.\2.ffn.inner_proj.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layers\.([0-9]+)\.fc2\.": r"encoder.layers.\2.ffn.output_proj.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layers\.([0-9]+)\.final_layer_norm\.": r"encoder.layers.\2.ffn_layer_norm.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.layer_norm\.": r"encoder.layer_norm.",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.pos_conv\.0\.weight_g$": r"encoder_frontend.pos_encoder.conv.parametrizations.weight.original0",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.pos_conv\.0\.weight_v$": r"encoder_frontend.pos_encoder.conv.parametrizations.weight.original1",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.pos_conv\.0\.bias$": r"encoder_frontend.pos_encoder.conv.bias",
    r"^(w2v_encoder\.w2v_model\.)?encoder\.pos_conv\.([0-4])\.0\.": r"encoder_frontend.pos_encoder.layers.\2.conv.",
    r"^(w2v_encoder\.w2v_model\.)?feature_extractor\.conv_layers\.([0-9]+)\.0\.": r"encoder_frontend.feature_extractor.layers.\2.conv.",
    r"^(w2v_encoder\.w2v_model\.)?feature_extractor\.conv_layers\.([0-9]+)\.2\.1\.": r"encoder_frontend.feature_extractor.layers.\2.layer_norm.",
    r"^(w2v_encoder\.w2v_model\.)?feature_extractor\.conv_layers\.0\.2\.": r"encoder_frontend.feature_extractor.layers.0.group_norm.",
    r"^(w2v_encoder\.w2v_model\.)?layer_norm\.": r"encoder_frontend.post_extract_layer_norm.",
    r"^(w2v_encoder\.w2v_model\.)?post_extract_proj\.": r"encoder_frontend.model_dim_proj.",
    r"^(w2v_encoder\.w2v_model\.)?mask_emb$": r"masker.temporal_mask_embed",
    r"^quantizer\.vars$": r"quantizer.entries",
    r"^quantizer\.weight_proj\.": r"quantizer.entry_proj.",
    r"^project_q\.": r"final_target_proj.",
    r"^w2v_encoder\.proj\.": r"final_proj.",
}


_HG = {
    r"^wav2vec2\.feature_extractor\.conv_layers\.([0-9]+)\.conv\.": r"encoder_frontend.feature_extractor.layers.\1.conv.",
    r"^wav2vec2\.feature_extractor\.conv_layers\.0\.layer_norm\.": r"encoder_frontend.feature_extractor.layers.0.@norm@.",
    r"^wav2vec2\.feature_extractor\.conv_layers\.([0-9]+)\.layer_norm\.": r"encoder_frontend.feature_extractor.layers.\1.layer_norm.",
    r"^wav2vec2\.feature_projection\.layer_norm\.": r"encoder_frontend.post_extract_layer_norm.",
    r"^wav2vec2\.feature_projection\.projection\.": r"encoder_frontend.model_dim_proj.",
    r"^wav2vec2\.encoder\.pos_conv_embed\.conv\.": r"encoder_frontend.pos_encoder.conv.",
    r"^wav2vec2\.encoder\.layer_norm\.": r"encoder.layer_norm.",
    r"^wav2vec2\.encoder\.layers\.([0-9]+)\.attention\.out_proj\.": r"encoder.layers.\1.self_attn.output_proj.",
    r"^wav2vec2\.encoder\.layers\.([0-9]+)\.attention\.(q|k|v)_proj\.": r"encoder.layers.\1.self_attn.\2_proj.",
    r"^wav2vec2\.encoder\.layers\.([0-9]+)\.layer_norm\.": r"encoder.layers.\1.self_attn_layer_norm.",
    r"^wav2vec2\.encoder\.layers\.([0-9]+)\.feed_forward\.intermediate_dense\.": r"encoder.layers.\1.ffn.inner_proj.",
    r"^wav2vec2\.encoder\.layers\.([0-9]+)\.feed_forward\.output_dense\.": r"encoder.layers.\1.ffn.output_proj.",
    r"^wav2vec2\.encoder\.layers\.([0-9]+)\.final_layer_norm\.": r"encoder.layers.\1.ffn_layer_norm.",
    r"^wav2vec2\.masked_spec_embed$": r"masker.temporal_mask_embed",
    r"^lm_head\.": r"final_proj.",
}


def _convert_hg(sd: dict[str, Any], norm_order: TransformerNormOrder, layer_norm_convs: bool) -> dict[str, Any]:
    out = convert_state_dict(sd, _HG)
    out = {k.replace("@norm@", "layer_norm" if layer_norm_convs else "group_norm"): v for k, v in out.items()}
    if norm_order == TransformerNormOrder.POST:
        for p in ("weight", "bias"):
            v = out.pop(f"encoder.layer_norm.{p}", None)
            if v is not None:
                out[f"encoder_frontend.layer_norm.{p}"] = v
    return out


def _convert(sd: dict[str, Any], norm_order: TransformerNormOrder, asr: bool, layer_norm_convs: bool = False
             ) -> dict[str, Any]:
    sd = dict(sd.get("model", sd))
    if any(k.startswith("wav2vec2.") for k in sd):
        return _convert_hg(sd, norm_order, layer_norm_convs)
    fairseq = any(k.endswith("mask_emb") or "conv_layers" in k for k in sd)
    if not fairseq:
        return {k.removeprefix("module."): v for k, v in sd.items()}
    out = convert_state_dict(sd, _COMMON)
    out = {k: v for k, v in out.items() if not k.endswith("version") and not k.endswith("_float_tensor")
           and not k.startswith("w2v_encoder.w2v_model.")}
    if norm_order == TransformerNormOrder.POST:
        # fairseq applies the embedding layer norm inside the encoder; here it belongs to the front end
        for p in ("weight", "bias"):
            v = out.pop(f"encoder.layer_norm.{p}", None)
            if v is not None:
                out[f"encoder_frontend.layer_norm.{p}"] = v
    if asr:
        for k in [k for k in out if k.startswith(("quantizer.", "final_target_proj.", "project_q."))]:
            del out[k]
    else:
        out["quantizer.num_updates"] = torch.zeros((), dtype=torch.int64)
    return out


def convert_wav2vec2_state_dict(sd: dict[str, Any], config: Any) -> dict[str, Any]:
    return _convert(sd, config.encoder_config.norm_order, False, config.encoder_config.feature_extractor_layer_norm_convs)


def convert_wav2vec2_asr_state_dict(sd: dict[str, Any], config: Any) -> dict[str, Any]:
    return _convert(sd, config.encoder_config.norm_order, True, config.encoder_config.feature_extractor_layer_norm_convs)
