"""Key map shared by the converters of original fairseq encoder-decoder checkpoints."""
from __future__ import annotations

from typing import Any, Mapping

from fairseq2_b200.models.llama.interop import convert_state_dict

FAIRSEQ_ENC_DEC_KEY_MAP = {
    r"^encoder\.embed_tokens\.": r"encoder_frontend.embed.",
    r"^decoder\.embed_tokens\.": r"decoder_frontend.embed.",
    r"^encoder\.layernorm_embedding\.": r"encoder_frontend.layer_norm.",
    r"^decoder\.layernorm_embedding\.": r"decoder_frontend.layer_norm.",
    r"^(encoder|decoder)\.layers\.([0-9]+)\.self_attn\.out_proj\.": r"\1.layers.\2.self_attn.output_proj.",
    r"^decoder\.layers\.([0-9]+)\.encoder_attn\.out_proj\.": r"decoder.layers.\1.encoder_decoder_attn.output_proj.",
    r"^decoder\.layers\.([0-9]+)\.encoder_attn\.": r"decoder.layers.\1.encoder_decoder_attn.",
    r"^decoder\.layers\.([0-9]+)\.encoder_attn_layer_norm\.": r"decoder.layers.\1.encoder_decoder_attn_layer_norm.",
    r"^(encoder|decoder)\.layers\.([0-9]+)\.fc1\.": r"\1.layers.\2.ffn.inner_proj.",
    r"^(encoder|decoder)\.layers\.([0-9]+)\.fc2\.": r"\1.layers.\2.ffn.output_proj.",
    r"^(encoder|decoder)\.layers\.([0-9]+)\.final_layer_norm\.": r"\1.layers.\2.ffn_layer_norm.",
    r"^decoder\.output_projection\.": r"final_proj.",
}

_DROP_SUFFIXES = ("version", "_float_tensor", "embed_positions._float_tensor")


def convert_fairseq_state_dict(sd: Mapping[str, Any], key_map: Mapping[str, str]) -> dict[str, Any]:
    """Unwraps ``{"model": ...}``, renames by ``key_map`` and drops fairseq bookkeeping entries."""
    sd = sd.get("model", sd)  # type: ignore[assignment]
    out = convert_state_dict(sd, key_map)
    return {k: v for k, v in out.items() if not k.endswith(_DROP_SUFFIXES)}
