"""Training engine.

Capability parity with fairseq2's ``Trainer`` (``trainer.py:105-1221``): a
``TrainUnit`` turns a batch into ``(loss, num_targets)``; the trainer runs the
state machine DATA_LOAD -> STEP -> POST_STEP with gradient accumulation,
``no_sync``, loss normalisation by the global number of targets, gradient
clipping, optimizer + LR scheduler stepping, fp16 loss scaling with overflow
retry, metric publishing, validation, checkpointing (with resume), early
stopping, graceful stop requests and profiler/GC hooks.

B200-first differences: the step never synchronises with the host -- the
normalisation factor, clip coefficient and gradient norm are device scalars
that feed the fused optimizer launch; step time is measured with CUDA events
(``DeviceStopwatch``) and read only when metrics are published.

``TrainStep`` is the reusable inner step (what ``bench.py`` times);
``Trainer`` drives it over a data reader.
"""
from __future__ import annotations

import signal
from abc import ABC, abstractmethod
from contextlib import nullcontext
from enum import Enum
from typing import Any, Generic, Iterable, Iterator, Mapping, Protocol, Sequence, TypeVar

import torch
from torch import Tensor
from torch.optim import Optimizer
from torch.profiler import record_function

from fairseq2_b200.error import InternalError, InvalidOperationError
from fairseq2_b200.gang import Gangs, ReduceOperation, broadcast_flag
from fairseq2_b200.logging import log
from fairseq2_b200.nn.data_parallel import DataParallelFacade
from fairseq2_b200.task import Task, TaskStopException
from fairseq2_b200.utils.rng import RngBag
from fairseq2_b200.utils.stopwatch import DeviceStopwatch, Stopwatch

BatchT = TypeVar("BatchT")


class TrainUnit(ABC, Generic[BatchT]):
    """Computes the loss of one batch (cf. reference ``trainer.py:69``)."""

    @abstractmethod
    def process_batch(self, batch: BatchT, metric_bag: Any | None = None) -> tuple[Tensor, int | Tensor | None]:
        """Returns ``(sum-reduced loss, number of targets)``; ``None`` targets
        means the loss is already a mean and must not be normalised."""

    def set_step_nr(self, step_nr: int) -> None:
        pass

    def set_data_epoch_nr(self, data_epoch_nr: int) -> None:
        pass

    def finalize(self, metric_bag: Any) -> None:
        pass

    @property
    @abstractmethod
    def model(self) -> DataParallelFacade: ...


class TrainStep:
    """One optimizer step over a list of micro-batches."""

    def __init__(self, unit: TrainUnit[Any], optimizer: Optimizer, gangs: Gangs, *, max_grad_norm: float | None = None,
                 lr_scheduler: Any | None = None, loss_scaler: Any | None = None, no_sync: bool = False,
                 metric_bag: Any | None = None) -> None:
        self.unit, self.optimizer, self.gangs = unit, optimizer, gangs
        self.max_grad_norm, self.lr_scheduler, self.loss_scaler = max_grad_norm, lr_scheduler, loss_scaler
        self.no_sync = no_sync
        self.metric_bag = metric_bag

    def __call__(self, batches: Sequence[Any], step_nr: int = 0) -> tuple[Tensor, Tensor]:
        """Returns ``(summed loss, gradient norm)`` as device tensors."""
        model = self.unit.model
        model.zero_grad()
        n = len(batches)
        total_loss: Tensor | None = None
        total_targets: Tensor | int | None = 0
        for i, batch in enumerate(batches):
            sync_ctx = model.no_sync() if (self.no_sync and i < n - 1) else nullcontext()
            with sync_ctx:
                with record_function(f"step_{step_nr}_{i}_forward"):
                    loss, num_targets = self.unit.process_batch(batch, self.metric_bag)
                with record_function(f"step_{step_nr}_{i}_backward"):
                    if self.loss_scaler is not None:
                        self.loss_scaler.backward(loss)
                    else:
                        loss.backward()
            total_loss = loss.detach() if total_loss is None else total_loss + loss.detach()
            if num_targets is None:
                total_targets = None
            elif total_targets is not None:
                total_targets = total_targets + num_targets
        model.finish_backward()
        assert total_loss is not None
        # ---- normalise: gradients hold the data-parallel MEAN of per-rank sums
        dp = self.gangs.dp
        if total_targets is not None:
            t = total_targets if isinstance(total_targets, Tensor) else \
                torch.tensor(float(total_targets), device=total_loss.device)
            t = t.to(torch.float32)
            if dp.size > 1:
                t = t.clone()
                dp.all_reduce(t, ReduceOperation.SUM)
            model.scale_grads(dp.size / t.clamp(min=1.0))
        elif n > 1:
            model.scale_grads(1.0 / n)
        if self.loss_scaler is not None:
            self.loss_scaler.unscale_grads_(model)
        with record_function(f"step_{step_nr}_grad_norm"):
            grad_norm = model.clip_grad_norm(self.max_grad_norm)
        with record_function(f"step_{step_nr}_optimizer"):
            scale = model.grad_scale
            if self.loss_scaler is not None:
                self.loss_scaler.run_optimizer_step(self.optimizer, grad_scale=scale)
            elif scale is not None:
                self.optimizer.step(grad_scale=scale)  # type: ignore[call-arg]
            else:
                self.optimizer.step()
            model.after_optimizer_step()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        return total_loss, grad_norm
