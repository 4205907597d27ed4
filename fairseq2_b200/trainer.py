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
from fairseq2_b200.validator import NoopValidator, Validator

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
                 metric_bag: Any | None = None, fuse_optimizer: bool = True) -> None:
        """``fuse_optimizer``: when nothing needs all gradients before the update (no gradient clipping, no loss
        scaler, one micro-batch) and the unit can tell its number of targets up front (``unit.count_targets``),
        the optimizer step of every FSDP unit runs inside its gradient reduce-scatter kernel."""
        self.fuse_optimizer = fuse_optimizer
        self.unit, self.optimizer, self.gangs = unit, optimizer, gangs
        self.max_grad_norm, self.lr_scheduler, self.loss_scaler = max_grad_norm, lr_scheduler, loss_scaler
        self.no_sync = no_sync
        self.metric_bag = metric_bag
        #: outcome of the last optimizer step under fp16 loss scaling (``None`` without a loss scaler)
        self.last_scale_result: Any | None = None

    def __call__(self, batches: Sequence[Any], step_nr: int = 0) -> tuple[Tensor, Tensor]:
        """Returns ``(summed loss, gradient norm)`` as device tensors."""
        model = self.unit.model
        # a collective kernel of an earlier step that gave up on a peer (bounded wait) surfaces here, before new
        # work is queued; the optimizer kernels skip their update on the device in the meantime
        check = getattr(model, "check_comm_status", None)
        if check is not None:
            check()
        model.zero_grad()
        n = len(batches)
        fused = self._maybe_arm_fused_optimizer(model, batches)
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
        if fused is not None:
            # the factor already went into the fused reduce-scatter + update kernels; units that were not armed
            # (rank-local ones, units outside a symmetric arena) get it through the regular optimizer launch
            model.scale_grads(fused)
        elif total_targets is not None:
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
                res = self.loss_scaler.run_optimizer_step(self.optimizer, grad_scale=scale, grad_norm=grad_norm)
                self.last_scale_result = res
                if res.overflowed:
                    # the step did not happen: weights, optimizer state and learning-rate schedule stay where they
                    # were and the caller repeats the batch with the reduced loss scale
                    return total_loss, grad_norm
            elif scale is not None:
                self.optimizer.step(grad_scale=scale)  # type: ignore[call-arg]
            else:
                self.optimizer.step()
            model.after_optimizer_step()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        if check is not None:
            check()
        return total_loss, grad_norm


def _arm_fused(self: TrainStep, model: Any, batches: Sequence[Any]) -> Tensor | None:
    """Returns the loss-normalisation factor (a device scalar) if the optimizer was armed, else ``None``."""
    count = getattr(self.unit, "count_targets", None)
    inner = getattr(model, "module", None)
    prepare = getattr(self.optimizer, "prepare_fused_step", None)
    if (not self.fuse_optimizer or count is None or prepare is None or len(batches) != 1
            or self.max_grad_norm is not None or self.loss_scaler is not None
            or not getattr(inner, "supports_fused_optimizer", False)):
        return None
    t = count(batches[0])
    dev = self.gangs.root.device
    t = t.to(device=dev, dtype=torch.float32) if isinstance(t, Tensor) else torch.tensor(float(t), device=dev)
    dp = self.gangs.dp
    if dp.size > 1:
        t = t.clone()
        dp.all_reduce(t, ReduceOperation.SUM)
    scale = dp.size / t.clamp(min=1.0)
    return scale if prepare(scale) > 0 else None


TrainStep._maybe_arm_fused_optimizer = _arm_fused  # type: ignore[attr-defined]


class _State(Enum):
    NOT_STARTED = 0
    DATA_LOAD = 1
    STEP = 2
    POST_STEP = 3
    END_OF_DATA_EPOCH = 4
    END_OF_TRAINING = 5
    END_OF_DATA = 6
    GRADIENT_OVERFLOW = 7
    EARLY_STOP = 8
    STOP_REQUESTED = 9
    STOPPED = 10


class MinimumLossScaleReachedError(Exception):
    def __init__(self, step_nr: int) -> None:
        super().__init__(f"The gradients are scaled down to the minimum loss scale at step {step_nr}; training cannot continue.")
        self.step_nr = step_nr


class InconsistentGradNormError(Exception):
    def __init__(self, step_nr: int) -> None:
        super().__init__(f"The gradient norms of the processes differ at step {step_nr}.")
        self.step_nr = step_nr


class Trainer(Task):
    """Drives a :class:`TrainUnit` over a data reader (reference ``trainer.py:105``)."""

    def __init__(self, *, unit: TrainUnit[Any], data_reader: Any, gangs: Gangs, optimizer: Optimizer,
                 lr_scheduler: Any | None = None, loss_scaler: Any | None = None, max_grad_norm: float | None = None,
                 no_sync_grad_accumulation: bool = False, grad_check: bool = False, seed: int = 2,
                 max_num_steps: int | None = None, max_num_data_epochs: int | None = None,
                 validator: Validator | None = None, validate_at_start: bool = False,
                 validate_after_n_steps: int = 0, validate_every_n_steps: int | None = None,
                 validate_every_n_data_epochs: int | None = None, early_stopper: Any | None = None,
                 checkpoint_manager: Any | None = None, checkpoint_after_n_steps: int = 0,
                 checkpoint_every_n_steps: int | None = None, checkpoint_every_n_data_epochs: int | None = None,
                 save_model_only: bool | str = False, keep_last_n_checkpoints: int | None = None,
                 keep_best_n_checkpoints: int | None = None, keep_checkpoint_every_n_steps: int | None = None,
                 metric_recorder: Any | None = None, publish_metrics_after_n_steps: int = 0,
                 publish_metrics_every_n_steps: int | None = None,
                 publish_metrics_every_n_data_epochs: int | None = None, profiler: Any | None = None,
                 garbage_collector: Any | None = None, device_stat_tracker: Any | None = None,
                 anomaly_detection: bool = False, wall_watch: Stopwatch | None = None,
                 hg_exporter: Any | None = None, fuse_optimizer: bool = True) -> None:
        from fairseq2_b200.metrics import MetricBag

        self._unit, self._reader, self._gangs = unit, data_reader, gangs
        self._optimizer, self._lr_scheduler, self._loss_scaler = optimizer, lr_scheduler, loss_scaler
        self._grad_check = grad_check
        self._seed = seed
        self._max_num_steps, self._max_num_data_epochs = max_num_steps, max_num_data_epochs
        self._validator = validator or NoopValidator()
        self._validate_at_start = validate_at_start
        self._validate_after_n_steps, self._validate_every_n_steps = validate_after_n_steps, validate_every_n_steps
        self._validate_every_n_data_epochs = validate_every_n_data_epochs
        self._early_stopper = early_stopper
        self._ckpt = checkpoint_manager
        self._ckpt_after, self._ckpt_every = checkpoint_after_n_steps, checkpoint_every_n_steps
        self._ckpt_every_epochs = checkpoint_every_n_data_epochs
        self._save_model_only = save_model_only
        self._keep_last_n, self._keep_best_n = keep_last_n_checkpoints, keep_best_n_checkpoints
        self._keep_every_n = keep_checkpoint_every_n_steps
        self._recorder = metric_recorder
        self._publish_after, self._publish_every = publish_metrics_after_n_steps, publish_metrics_every_n_steps
        self._publish_every_epochs = publish_metrics_every_n_data_epochs
        self._profiler, self._gc, self._stat = profiler, garbage_collector, device_stat_tracker
        self._anomaly_detection = anomaly_detection
        self._hg_exporter = hg_exporter
        device = gangs.root.device
        self._device = device
        self._metric_bag = MetricBag(device)
        self._step_fn = TrainStep(unit, optimizer, gangs, max_grad_norm=max_grad_norm, lr_scheduler=lr_scheduler,
                                  loss_scaler=loss_scaler, no_sync=no_sync_grad_accumulation,
                                  metric_bag=self._metric_bag, fuse_optimizer=fuse_optimizer)
        self._rng_bag = RngBag.from_device_defaults(torch.device("cpu"), device) if device.type == "cuda" \
            else RngBag.from_device_defaults(device)
        self._state = _State.NOT_STARTED
        self._step_nr = 0
        self._data_epoch_nr = 1
        self._batches: list[Any] | None = None
        self._stop_requested = False
        self._has_read_any = False
        self._best_score: float | None = None
        self._wall_watch = wall_watch or Stopwatch()
        if not self._wall_watch.is_running:
            self._wall_watch.start()
        self._base_wall_time = 0.0
        self._total_watch = Stopwatch()
        self._data_watch = Stopwatch()
        self._compute_watch = DeviceStopwatch(device)
        self._lapse_watch = Stopwatch()
        self._num_batches_read = 0
        self._last_grad_norm: Tensor | None = None
        self._last_loss: Tensor | None = None

    # -------------------------------------------------------------- interface
    @property
    def step_nr(self) -> int:
        return self._step_nr

    def request_stop(self) -> None:
        log.info("Stop requested; training will stop after the current step.")
        self._stop_requested = True

    def close(self) -> None:
        if self._recorder is not None:
            self._recorder.close()
        if self._ckpt is not None:
            self._ckpt.close()
        if self._hg_exporter is not None:
            self._hg_exporter.complete_pending_export_operations(blocking=True)
        self._validator.close()

    def run(self) -> None:
        if self._state != _State.NOT_STARTED:
            raise InvalidOperationError("The trainer can only be run once.")
        g = self._gangs
        self._rng_bag.manual_seed(self._seed + g.root.rank)
        self._maybe_restore_state()
        prof = self._profiler if self._profiler is not None else nullcontext()
        gc_ctx = self._gc if self._gc is not None and hasattr(self._gc, "__enter__") else nullcontext()
        anomaly = torch.autograd.set_detect_anomaly(True, check_nan=True) if self._anomaly_detection else nullcontext()
        self._unit.model.train(True)
        self._total_watch.start()
        self._lapse_watch.start()
        log.info("Training started at step {}.", self._step_nr)
        try:
            with prof, gc_ctx, anomaly:
                self._do_run()
        except KeyboardInterrupt:
            log.info("Training interrupted at step {}.", self._step_nr)
            raise
        finally:
            self._total_watch.stop()
        if self._state == _State.STOPPED:
            raise TaskStopException()
        log.info("Training finished at step {} after {:.0f} second(s).", self._step_nr,
                 self._total_watch.get_elapsed_time())

    # ------------------------------------------------------------ state machine
    def _do_run(self) -> None:
        if self._validate_at_start and self._step_nr == 0:
            self._validate()
        self._state = _State.DATA_LOAD
        while True:
            st = self._state
            if st == _State.DATA_LOAD:
                self._state = self._read_next_batches()
            elif st == _State.STEP:
                self._state = self._run_step()
            elif st == _State.POST_STEP:
                self._state = self._post_step()
            elif st == _State.END_OF_DATA_EPOCH:
                self._state = self._end_of_data_epoch()
            elif st == _State.GRADIENT_OVERFLOW:
                self._state = _State.STEP      # retry the same batches with the reduced loss scale
            elif st in (_State.END_OF_TRAINING, _State.END_OF_DATA, _State.EARLY_STOP):
                self._finish(blocking=True)
                return
            elif st == _State.STOP_REQUESTED:
                self._finish(blocking=True)
                self._state = _State.STOPPED
                return
            else:
                raise InternalError(f"Unexpected trainer state {st}.")

    def _read_next_batches(self) -> _State:
        self._data_watch.start()
        try:
            self._batches = next(self._reader)
            self._has_read_any = True
            self._num_batches_read += len(self._batches)
        except StopIteration:
            self._batches = None
        finally:
            self._data_watch.stop()
        if self._batches is None:
            return _State.END_OF_DATA_EPOCH
        return _State.STEP

    def _end_of_data_epoch(self) -> _State:
        if not self._has_read_any:
            log.info("The data reader produced no batch; training ends.")
            return _State.END_OF_DATA
        log.info("End of data epoch {} reached at step {}.", self._data_epoch_nr, self._step_nr)
        epoch = self._data_epoch_nr
        if self._should_do_every_epochs(self._publish_every_epochs, epoch):
            self._publish_metrics()
        if self._should_do_every_epochs(self._validate_every_n_data_epochs, epoch):
            self._validate()
        if self._should_do_every_epochs(self._ckpt_every_epochs, epoch):
            self._save_checkpoint(blocking=False)
        if self._max_num_data_epochs is not None and epoch >= self._max_num_data_epochs:
            return _State.END_OF_TRAINING
        self._data_epoch_nr += 1
        self._unit.set_data_epoch_nr(self._data_epoch_nr)
        self._reader.reset()
        self._has_read_any = False
        return _State.DATA_LOAD

    @staticmethod
    def _should_do_every_epochs(every: int | None, epoch: int) -> bool:
        return every is not None and epoch % every == 0

    def _run_step(self) -> _State:
        assert self._batches is not None
        step_nr = self._step_nr + 1
        self._unit.set_step_nr(step_nr)
        self._metric_bag.begin_updates()
        batches = [b.to(self._device, non_blocking=True) if hasattr(b, "to") else b for b in self._batches]
        self._compute_watch.start()
        with record_function(f"step_{step_nr}"):
            try:
                loss, grad_norm = self._step_fn(batches, step_nr)
            except torch.OutOfMemoryError:
                log.error("CUDA ran out of memory at step {}. Batch shapes: {}", step_nr,
                          [getattr(getattr(b, 'seqs', None), 'shape', None) for b in batches])
                raise
        self._compute_watch.stop()
        res = self._step_fn.last_scale_result
        if res is not None and res.overflowed:
            self._metric_bag.rollback_updates()
            if res.exploded:
                raise MinimumLossScaleReachedError(step_nr)
            return _State.GRADIENT_OVERFLOW
        if self._grad_check:
            from fairseq2_b200.nn.utils.grad import check_grad_norms

            if not check_grad_norms(grad_norm, self._gangs.dp, step_nr):
                raise InconsistentGradNormError(step_nr)
        self._metric_bag.commit_updates()
        from fairseq2_b200.metrics import Mean

        self._metric_bag.get("grad_norm", Mean).update(grad_norm)
        self._last_grad_norm, self._last_loss = grad_norm, loss
        self._step_nr = step_nr
        self._batches = None
        if self._profiler is not None:
            self._profiler.step()
        if self._gc is not None:
            self._gc.step()
        return _State.POST_STEP

    def _post_step(self) -> _State:
        step = self._step_nr
        if self._ckpt is not None:
            self._ckpt.maybe_complete_save_operation(blocking=False)
        if self._should_do(step, self._publish_after, self._publish_every):
            self._publish_metrics()
        stop = False
        if self._should_do(step, self._validate_after_n_steps, self._validate_every_n_steps):
            stop = self._validate()
        if self._should_do(step, self._ckpt_after, self._ckpt_every):
            self._save_checkpoint(blocking=False)
        if stop:
            return _State.EARLY_STOP
        if self._max_num_steps is not None and step >= self._max_num_steps:
            return _State.END_OF_TRAINING
        if self._stop_requested:
            return _State.STOP_REQUESTED
        return _State.DATA_LOAD

    @staticmethod
    def _should_do(step: int, after: int, every: int | None) -> bool:
        return every is not None and step >= after and step % every == 0

    def _finish(self, blocking: bool) -> None:
        if self._publish_every is not None and self._step_nr % self._publish_every != 0:
            self._publish_metrics()
        if self._ckpt is not None and (self._ckpt_every is not None or self._ckpt_every_epochs is not None):
            self._ckpt.maybe_complete_save_operation(blocking=True)
            last = self._ckpt.maybe_get_last_step_number()
            if last != self._step_nr and self._step_nr > 0:
                self._save_checkpoint(blocking=True)
            self._ckpt.maybe_complete_save_operation(blocking=True)

    # ---------------------------------------------------------------- metrics
    def _publish_metrics(self) -> None:
        from fairseq2_b200.metrics import sync_and_compute_metrics
        from fairseq2_b200.metrics.common import extend_batch_metric_values

        g = self._gangs
        values = sync_and_compute_metrics(self._metric_bag, g.dp) if g.tp.rank == 0 else None
        self._unit.finalize(self._metric_bag)
        self._metric_bag.reset_non_persistent_metrics()
        compute_time = self._compute_watch.get_elapsed_time()
        data_time = self._data_watch.get_elapsed_time()
        lapse = self._lapse_watch.get_elapsed_time()
        if g.root.rank == 0 and values is not None:
            if self._lr_scheduler is not None:
                values["lr"] = float(self._lr_scheduler.get_last_lr()[0])
            else:
                values["lr"] = float(self._optimizer.param_groups[0]["lr"])
            values["data_epoch"] = self._data_epoch_nr
            values["data_time"], values["compute_time"], values["lapse_time"] = data_time, compute_time, lapse
            values["total_time"] = self._total_watch.get_elapsed_time()
            values["wall_time"] = self._base_wall_time + self._wall_watch.get_elapsed_time()
            extend_batch_metric_values(values, self._num_batches_read * g.dp.size, compute_time + data_time)
            if self._stat is not None:
                values.update(self._stat.get_stats())
            if self._recorder is not None:
                self._recorder.record_metric_values("train", values, self._step_nr)
        if self._stat is not None:
            self._stat.reset_stats()
        self._compute_watch.reset()
        self._data_watch.reset()
        self._lapse_watch.reset()
        self._num_batches_read = 0
        g.root.barrier()

    # ------------------------------------------------------------- validation
    def _validate(self) -> bool:
        self._unit.model.train(False)
        try:
            score = self._validator.run(self._step_nr)
        finally:
            self._unit.model.train(True)
        self._validator.reset()
        stop = False
        if score is not None:
            if self._best_score is None or score > self._best_score:
                self._best_score = score
            if self._ckpt is not None:
                self._ckpt.save_score(self._step_nr, score)
            if self._early_stopper is not None:
                g = self._gangs
                flag = self._early_stopper.should_stop(self._step_nr, score) if g.root.rank == 0 else False
                stop = broadcast_flag(g.root, flag)
                if stop:
                    log.info("Early stop at step {}.", self._step_nr)
        return stop

    # ------------------------------------------------------------ checkpoints
    def state_dict(self) -> dict[str, Any]:
        sd: dict[str, Any] = {
            "_step_nr": self._step_nr, "_data_epoch_nr": self._data_epoch_nr,
            "_rng_bag": self._rng_bag.state_dict(), "_metric_bag": self._metric_bag.state_dict(),
            "_base_wall_time": self._base_wall_time + self._wall_watch.get_elapsed_time(),
            "_best_score": self._best_score,
            # whether the current data epoch has produced a batch: a run that resumes exactly at the end of an epoch
            # reads nothing before the reader reports the end, and must not mistake that for an empty dataset
            "_has_read_any": self._has_read_any,
        }
        if self._lr_scheduler is not None:
            sd["_lr_scheduler"] = self._lr_scheduler.state_dict()
        if self._loss_scaler is not None:
            sd["_fp16_loss_scaler"] = self._loss_scaler.state_dict()
        return sd

    def load_state_dict(self, sd: Mapping[str, Any]) -> None:
        self._step_nr = int(sd["_step_nr"])
        self._data_epoch_nr = int(sd["_data_epoch_nr"])
        self._rng_bag.load_state_dict(sd["_rng_bag"])
        self._metric_bag.load_state_dict(sd.get("_metric_bag", {}))
        self._base_wall_time = float(sd.get("_base_wall_time", 0.0))
        self._best_score = sd.get("_best_score")
        self._has_read_any = bool(sd.get("_has_read_any", self._step_nr > 0))
        if self._lr_scheduler is not None and "_lr_scheduler" in sd:
            self._lr_scheduler.load_state_dict(sd["_lr_scheduler"])
        if self._loss_scaler is not None and "_fp16_loss_scaler" in sd:
            self._loss_scaler.load_state_dict(sd["_fp16_loss_scaler"])

    def _save_checkpoint(self, blocking: bool) -> None:
        if self._ckpt is None:
            return
        step = self._step_nr
        log.info("Saving the checkpoint of step {}.", step)
        model_only = self._save_model_only is True or self._save_model_only == "all" or \
            (self._save_model_only == "all_but_last" and False)
        cb = self._checkpoint_saved
        if model_only:
            self._ckpt.save_model_only(step, self._unit.model, callback=cb, blocking=blocking)
        else:
            self._ckpt.save_checkpoint(step, self, self._unit.model, self._optimizer, self._reader, callback=cb,
                                       blocking=blocking)

    def _checkpoint_saved(self, step_nr: int) -> None:
        if self._ckpt is None:
            return
        if self._keep_last_n is not None or self._keep_best_n is not None:
            self._ckpt.delete_stale_checkpoints(keep_last_n=self._keep_last_n, keep_best_n=self._keep_best_n,
                                                keep_every_n_steps=self._keep_every_n,
                                                keep_model_only=self._save_model_only == "all_but_last")
        if self._hg_exporter is not None:
            self._hg_exporter.export(step_nr)

    def _maybe_restore_state(self) -> None:
        if self._ckpt is None:
            return
        step = self._ckpt.maybe_get_last_step_number(exclude_model_only=True)
        if step is None:
            return
        log.info("Restoring training from the checkpoint of step {}.", step)
        self._ckpt.load_trainer_state(step, self)
        self._ckpt.load_model_state(step, self._unit.model)
        self._ckpt.load_optimizer_state(step, self._optimizer)
        # A reader without position state (synthetic data) restarts from the beginning. That is decided from the
        # reader itself, identically on every rank; a missing or corrupt state FILE is an error that propagates
        # (the load contains a barrier, so swallowing it on one rank would leave the others waiting).
        if getattr(self._reader, "stateless", False):
            log.warning("The data reader keeps no position; the data restarts from the beginning at step {}.", step)
        else:
            self._ckpt.load_data_reader_state(step, self._reader)
        self._unit.set_step_nr(self._step_nr)
        self._unit.set_data_epoch_nr(self._data_epoch_nr)
        self._gangs.root.barrier()
        log.info("Training restored; resuming from step {}.", self._step_nr)


def install_stop_signal_handler(task: Task, signum: int = signal.SIGUSR1) -> None:
    """``SIGUSR1`` (what Slurm sends before preemption) requests a graceful stop."""
    def handler(sig: int, frame: Any) -> None:
        task.request_stop()

    signal.signal(signum, handler)
