"""Base of Trainer/Evaluator/Generator loops (cf. ``src/fairseq2/task.py``)."""
from __future__ import annotations

from abc import ABC, abstractmethod


class Task(ABC):
    @abstractmethod
    def run(self) -> None: ...

    @abstractmethod
    def request_stop(self) -> None: ...

    @abstractmethod
    def close(self) -> None: ...

    @property
    @abstractmethod
    def step_nr(self) -> int: ...


class TaskStopException(Exception):
    """Raised out of ``run()`` when a requested stop has completed."""
