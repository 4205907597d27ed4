"""Early-stopping protocol (cf. ``src/fairseq2/early_stopper.py``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import final


class EarlyStopper(ABC):
    @abstractmethod
    def should_stop(self, step_nr: int, score: float) -> bool: ...


@final
class NoopEarlyStopper(EarlyStopper):
    def should_stop(self, step_nr: int, score: float) -> bool:
        return False
