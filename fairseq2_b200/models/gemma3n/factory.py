"""Gemma 3n factory (cf. fairseq2 ``models/gemma3n/factory.py:40-432``)."""
from __future__ import annotations

from fairseq2_b200.gang import Gangs
from fairseq2_b200.models.gemma3n.config import Gemma3nConfig
from fairseq2_b200.models.gemma3n.model import Gemma3nModel


def create_gemma3n_model(config: Gemma3nConfig, gangs: Gangs | None = None) -> Gemma3nModel:
    if gangs is not None and gangs.tp.size > 1:
        raise NotImplementedError("Tensor parallelism is not implemented for Gemma 3n.")
    return Gemma3nModel(config)


def gemma3n_wrap_policy(module):  # type: ignore[no-untyped-def]
    """One FSDP unit per decoder layer."""
    return list(module.layers)
