"""Evaluation and generation loops (cf. fairseq2 ``evaluator.py:44-345``,
``validator.py:45-341``, ``generator.py:42-315``).

* :class:`EvalUnit` computes metrics of one batch into a metric bag.
* :class:`Evaluator` is the task that runs a list of ``(unit, data_reader)``
  pairs under ``no_grad`` + inference autocast and publishes the synced metrics.
* :class:`StandardValidator` is the same loop packaged as the trainer's
  validator; it derives a score (higher is better) from a named metric.
* :class:`GeneratorUnit`/:class:`Generator` run a generation job over a reader.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from contextlib import nullcontext
from typing import Any, Generic, Sequence, TypeVar

import torch

from fairseq2_b200.gang import Gangs
from fairseq2_b200.logging import log
from fairseq2_b200.metrics import MetricBag, sync_and_compute_metrics
from fairseq2_b200.metrics.common import extend_batch_metric_values
from fairseq2_b200.task import Task, TaskStopException
from fairseq2_b200.trainer import Validator
from fairseq2_b200.utils.progress import create_progress_reporter
from fairseq2_b200.utils.rng import RngBag
from fairseq2_b200.utils.stopwatch import Stopwatch

BatchT = TypeVar("BatchT")


class EvalUnit(ABC, Generic[BatchT]):
    @abstractmethod
    def process_batch(self, batch: BatchT, metric_bag: MetricBag) -> None: ...

    def prepare_metric_bag(self, metric_bag: MetricBag) -> None:
        """Called once before the first batch: register the metrics the unit will update."""

    def set_train_step_nr(self, train_step_nr: int) -> None:
        pass

    def finalize(self, metric_bag: MetricBag) -> None:
        pass

    def process_metric_values(self, values: dict[str, Any]) -> None:
        pass

    @property
    def name(self) -> str | None:
        return None

    @property
    @abstractmethod
    def model(self) -> Any: ...


class GeneratorUnit(EvalUnit[BatchT]):
    """Same contract as :class:`EvalUnit`; ``process_batch`` generates and writes its outputs."""


def _autocast(device: torch.device, amp: bool, dtype: torch.dtype) -> Any:
    return torch.autocast(device_type=device.type, dtype=dtype) if amp else nullcontext()


class _EvalLoop:
    def __init__(self, units: Sequence[EvalUnit[Any]], data_readers: Sequence[Any], gangs: Gangs, *,
                 amp: bool = False, amp_dtype: torch.dtype = torch.bfloat16, metric_recorder: Any | None = None,
                 device_stat_tracker: Any | None = None, category: str = "eval", seed: int = 2) -> None:
        if len(units) != len(data_readers):
            raise ValueError(f"The number of units ({len(units)}) must match the number of data readers "
                             f"({len(data_readers)}).")
        self._units, self._readers, self._gangs = list(units), list(data_readers), gangs
        self._amp, self._amp_dtype = amp, amp_dtype
        self._recorder, self._stat, self._category = metric_recorder, device_stat_tracker, category
        self._seed = seed
        self._step_nr = 0
        self._stop = False
        device = gangs.root.device
        self._rng_bag = RngBag.from_device_defaults(torch.device("cpu"), device) if device.type == "cuda" \
            else RngBag.from_device_defaults(device)

    def _run_unit(self, unit: EvalUnit[Any], reader: Any, train_step_nr: int | None) -> dict[str, Any] | None:
        g = self._gangs
        device = g.root.device
        bag = MetricBag(device)
        unit.prepare_metric_bag(bag)
        if train_step_nr is not None:
            unit.set_train_step_nr(train_step_nr)
        watch = Stopwatch()
        watch.start()
        num_batches = 0
        self._step_nr = 0
        module = unit.model.module if hasattr(unit.model, "module") else unit.model
        was_training = getattr(module, "training", False)
        module.train(False)
        label = self._category if unit.name is None else f"{self._category}/{unit.name}"
        task = create_progress_reporter().create_task(label, None) if g.root.rank == 0 else None
        try:
            # The random state of the surrounding job (dropout and masking of the training step that follows a
            # validation) must not depend on whether, or on how much data, was evaluated in between.
            with self._rng_bag.temporary_manual_seed(self._seed + g.root.rank), torch.no_grad(), \
                    _autocast(device, self._amp, self._amp_dtype):
                for batches in reader:
                    if self._stop:
                        raise TaskStopException()
                    self._step_nr += 1
                    for batch in batches:
                        if hasattr(batch, "to"):
                            batch = batch.to(device, non_blocking=True)
                        unit.process_batch(batch, bag)
                        num_batches += 1
                    if task is not None:
                        task.step(1)
        finally:
            if task is not None:
                task.close()
            module.train(was_training)
            reader.reset()
        values = sync_and_compute_metrics(bag, g.dp) if g.tp.rank == 0 else None
        unit.finalize(bag)
        elapsed = watch.get_elapsed_time()
        if values is not None:
            extend_batch_metric_values(values, num_batches * g.dp.size, elapsed)
            values["elapsed_time"] = elapsed
            if self._stat is not None:
                values.update(self._stat.get_stats())
            unit.process_metric_values(values)
            if g.root.rank == 0 and self._recorder is not None:
                cat = self._category if unit.name is None else f"{self._category}/{unit.name}"
                self._recorder.record_metric_values(cat, values, train_step_nr)
        if self._stat is not None:
            self._stat.reset_stats()
        g.root.barrier()
        return values


class Evaluator(Task, _EvalLoop):
    def __init__(self, units: Sequence[EvalUnit[Any]], data_readers: Sequence[Any], gangs: Gangs, **kw: Any) -> None:
        _EvalLoop.__init__(self, units, data_readers, gangs, **kw)
        self._ran = False
        self.results: list[dict[str, Any] | None] = []

    def run(self) -> None:
        if self._ran:
            raise RuntimeError("The evaluator can only be run once.")
        self._ran = True
        log.info("Evaluation starting.")
        for unit, reader in zip(self._units, self._readers):
            self.results.append(self._run_unit(unit, reader, None))
        log.info("Evaluation finished.")

    def request_stop(self) -> None:
        self._stop = True

    def close(self) -> None:
        if self._recorder is not None:
            self._recorder.close()

    @property
    def step_nr(self) -> int:
        return self._step_nr


class Generator(Evaluator):
    """The generation task: identical control flow, metrics published under ``generation``."""

    def __init__(self, unit: GeneratorUnit[Any], data_reader: Any, gangs: Gangs, **kw: Any) -> None:
        kw.setdefault("category", "generation")
        super().__init__([unit], [data_reader], gangs, **kw)


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
