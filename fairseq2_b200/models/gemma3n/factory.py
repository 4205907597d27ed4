"""Gemma 3n factory (cf. fairseq2 ``models/gemma3n/factory.py:40-432``): builds the text decoder (and the audio
tower when the config has one); with a tensor-parallel gang the attention heads and the FFN inner dimension are
split over it (see :mod:`fairseq2_b200.models.gemma3n.model`), the audio tower stays replicated."""
from __future__ import annotations

from fairseq2_b200.gang import Gangs
from fairseq2_b200.models.gemma3n.config import Gemma3nConfig
from fairseq2_b200.models.gemma3n.model import Gemma3nModel


def create_gemma3n_model(config: Gemma3nConfig, gangs: Gangs | None = None) -> Gemma3nModel:
    tp = gangs.tp if gangs is not None and gangs.tp.size > 1 else None
    if tp is not None:
        if config.num_attn_heads % tp.size or config.num_key_value_heads % tp.size:
            raise ValueError(
                f"The tensor parallel size ({tp.size}) must divide the number of attention heads "
                f"({config.num_attn_heads}) and of key-value heads ({config.num_key_value_heads}) of Gemma 3n.")
        if config.ffn_inner_dim % tp.size:
            raise ValueError(f"The tensor parallel size ({tp.size}) must divide `ffn_inner_dim` ({config.ffn_inner_dim}).")
    return Gemma3nModel(config, tp_gang=tp)


def gemma3n_wrap_policy(module):  # type: ignore[no-untyped-def]
    """One FSDP unit per decoder layer."""
    return list(module.layers)
