"""The generation task (cf. fairseq2 ``generator.py:69-268``): :class:`GeneratorUnit`s generate from the batches of
a data reader and write their outputs; :class:`Generator` runs them with the evaluation loop (inference mode,
autocast, metrics synced over the gangs and published under ``generation``)."""
from __future__ import annotations

from typing import Any

from fairseq2_b200.evaluator import BatchT, EvalUnit, Evaluator
from fairseq2_b200.gang import Gangs

__all__ = ["Generator", "GeneratorUnit"]


class GeneratorUnit(EvalUnit[BatchT]):
    """Same contract as :class:`EvalUnit`; ``process_batch`` generates and writes its outputs."""


class Generator(Evaluator):
    """The generation task: identical control flow, metrics published under ``generation``."""

    def __init__(self, unit: GeneratorUnit[Any], data_reader: Any, gangs: Gangs, **kw: Any) -> None:
        kw.setdefault("category", "generation")
        super().__init__([unit], [data_reader], gangs, **kw)
