"""Validation during training (cf. fairseq2 ``validator.py:69-419``): the :class:`Validator` interface that the
trainer calls every ``validate_every_n_steps``, and :class:`StandardValidator`, the evaluation loop over
``EvalUnit``s that derives the checkpoint score from a named metric and keeps track of the best one."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Sequence

import torch

from fairseq2_b200.evaluator import EvalUnit, _EvalLoop
from fairseq2_b200.gang import Gangs
from fairseq2_b200.logging import log

__all__ = ["EvalUnit", "NoopValidator", "StandardValidator", "Validator"]


class Validator(ABC):
    """Runs validation and returns a score (higher is better) or ``None``."""

    @abstractmethod
    def run(self, train_step_nr: int) -> float | None: ...

    def reset(self) -> None:
        pass

    def close(self) -> None:
        pass


class NoopValidator(Validator):
    def run(self, train_step_nr: int) -> float | None:
        return None


class StandardValidator(Validator, _EvalLoop):
    """Validation inside training. ``score_metric`` names the metric that becomes the checkpoint score;
    ``lower_better`` negates it so that a higher score is always better. The best score and its step are tracked
    across runs (and picked up from the scores of the saved checkpoints after a restart when a
    ``checkpoint_manager`` is given), and logged next to the last one."""

    def __init__(self, units: Sequence[EvalUnit[Any]], data_readers: Sequence[Any], gangs: Gangs, *,
                 score_metric: str | None = None, lower_better: bool = False, checkpoint_manager: Any | None = None,
                 **kw: Any) -> None:
        kw.setdefault("category", "valid")
        _EvalLoop.__init__(self, units, data_readers, gangs, **kw)
        self._score_metric, self._lower_better = score_metric, lower_better
        self._ckpt = checkpoint_manager
        self._best_score = float("-inf")
        self._best_step_nr = -1                     # -1: not yet compared with the checkpoints on disk

    @property
    def best_score(self) -> float | None:
        """The best score so far in the metric's own direction (``None`` before the first scored run)."""
        if self._best_step_nr <= 0:
            return None
        return -self._best_score if self._lower_better else self._best_score

    @property
    def best_step_nr(self) -> int | None:
        return self._best_step_nr if self._best_step_nr > 0 else None

    def _maybe_restore_best(self) -> None:
        if self._score_metric is None or self._best_step_nr >= 0:
            return
        self._best_step_nr = 0
        if self._ckpt is not None:
            scored = self._ckpt.load_scores()       # best first, higher is better
            if scored:
                self._best_score, self._best_step_nr = float(scored[0][0]), int(scored[0][1])

    def run(self, train_step_nr: int) -> float | None:
        log.info("Validation at step {} starting.", train_step_nr)
        self._maybe_restore_best()
        scores = []
        for unit, reader in zip(self._units, self._readers):
            if unit.name:
                log.info("Validating {}.", unit.name)
            values = self._run_unit(unit, reader, train_step_nr)
            if self._score_metric is not None and values is not None and self._score_metric in values:
                scores.append(float(values[self._score_metric]))
        score: float | None = None
        if self._score_metric is not None:
            g = self._gangs
            # the score is computed where tp.rank == 0 and shared so that every rank takes the same decisions
            t = torch.tensor([sum(scores) / len(scores) if scores else float("nan")], device=g.root.device,
                             dtype=torch.float64)
            g.root.broadcast(t, 0)
            v = float(t.item())
            if v == v:
                score = -v if self._lower_better else v
                if score > self._best_score:
                    self._best_score, self._best_step_nr = score, train_step_nr
                log.info("Score - Metric: {} | Last: {:.6g} (step {}) | Best: {:.6g} (step {})", self._score_metric, v,
                         train_step_nr, -self._best_score if self._lower_better else self._best_score,
                         self._best_step_nr)
        log.info("Validation finished.")
        return score

    def reset(self) -> None:
        self._step_nr = 0
        self._stop = False
        for reader in self._readers:
            reader.reset()

    def close(self) -> None:
        pass
