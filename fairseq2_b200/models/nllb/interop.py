"""Conversion of original fairseq NLLB checkpoints (cf. fairseq2 ``models/nllb/interop.py:21-75``)."""
from __future__ import annotations

from typing import Any

import torch

from fairseq2_b200.models.nllb.config import NllbConfig
from fairseq2_b200.models.utils_fairseq import FAIRSEQ_ENC_DEC_KEY_MAP, convert_fairseq_state_dict


def convert_nllb_state_dict(sd: dict[str, Any], config: NllbConfig) -> dict[str, Any]:
    inner = sd.get("model", sd)
    if "decoder.embed_tokens.weight" not in inner:
        return {k.removeprefix("module."): v for k, v in inner.items()}
    out = convert_fairseq_state_dict(sd, FAIRSEQ_ENC_DEC_KEY_MAP)
    embeds = out["final_proj.weight"]
    if embeds.size(0) == 256103:          # NLLB-100 carries one extra symbol at the end
        embeds = embeds[:-1]
    # fairseq orders the control symbols <s> <pad> </s> <unk>; here: <pad> <unk> <s> </s>
    embeds = embeds.clone()
    embeds[[0, 1, 2, 3]] = embeds[[1, 3, 0, 2]]
    out["encoder_frontend.embed.weight"] = embeds
    out.pop("decoder_frontend.embed.weight", None)
    out.pop("final_proj.weight", None)
    return out
