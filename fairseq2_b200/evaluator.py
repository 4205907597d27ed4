"""The evaluation task and the loop it shares with validation and generation (cf. fairseq2 ``evaluator.py:44-345``).

* :class:`EvalUnit` computes metrics of one batch into a metric bag.
* :class:`Evaluator` is the task that runs a list of ``(unit, data_reader)`` pairs under ``no_grad`` + inference
  autocast and publishes the synced metrics.
* ``_EvalLoop`` is that loop; :mod:`fairseq2_b200.validator` packages it as the trainer's validator and
  :mod:`fairseq2_b200.generator` as the generation task (both are re-exported here).
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


def __getattr__(name: str) -> Any:
    # the validator and the generator build on this module: resolve them lazily for importers of the old location
    if name == "StandardValidator":
        from fairseq2_b200.validator import StandardValidator

        return StandardValidator
    if name in ("Generator", "GeneratorUnit"):
        import fairseq2_b200.generator as g

        return getattr(g, name)
    raise AttributeError(f"module 'fairseq2_b200.evaluator' has no attribute '{name}'")
