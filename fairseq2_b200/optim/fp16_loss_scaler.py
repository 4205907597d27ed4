"""Dynamic loss scaling for fp16 training (cf. fairseq2
``optim/fp16_loss_scaler.py:28-317``): scale the loss, unscale gradients, skip
the step on overflow and halve the scale; double it after ``scale_window``
clean steps; give up below ``min_scale``. With bf16/fp32 a no-op scaler is
used. The found-inf flag is reduced over the gang so all ranks skip together."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

import torch
from torch import Tensor
from torch.optim import Optimizer

from fairseq2_b200.gang import Gang, ReduceOperation
from fairseq2_b200.logging import log


@dataclass(frozen=True)
class Float16LossScaleResult:
    old_scale: float
    new_scale: float
    overflowed: bool = False
    exploded: bool = False  # scale fell below `min_scale`


class Float16LossScaler:
    def backward(self, loss: Tensor) -> None:
        loss.backward()

    def unscale_grads_(self, model: Any) -> None:
        pass

    def run_optimizer_step(self, optimizer: Optimizer, *, grad_scale: Tensor | None = None,
                           grad_norm: Tensor | None = None) -> Float16LossScaleResult:
        if grad_scale is not None:
            optimizer.step(grad_scale=grad_scale)  # type: ignore[call-arg]
        else:
            optimizer.step()
        return Float16LossScaleResult(1.0, 1.0)

    def get_scale(self) -> float:
        return 1.0

    def state_dict(self) -> dict[str, Any]:
        return {}

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        pass


NoopFloat16LossScaler = Float16LossScaler


class StandardFloat16LossScaler(Float16LossScaler):
    def __init__(self, gang: Gang, *, init_scale: float = 2.0 ** 15, scale_factor: float = 2.0,
                 scale_window: int | None = None, min_scale: float = 0.0, gradient_accumulation: int = 1) -> None:
        if scale_window is None:
            # fairseq heuristic: the window shrinks with the number of workers and accumulated batches
            scale_window = max(int(2 ** 14 / gang.size / gradient_accumulation), 1)
        self._gang = gang
        self._scale = float(init_scale)
        self._factor, self._window, self._min_scale = scale_factor, scale_window, min_scale
        self._good_steps = 0
        self._found_inf: Tensor | None = None

    def backward(self, loss: Tensor) -> None:
        (loss * self._scale).backward()

    def unscale_grads_(self, model: Any) -> None:
        """Divides the gradients by the loss scale and looks for non-finite values. A model whose gradients live
        in flat shards and whose scaling is deferred into the optimizer launch (``scale_grads`` + ``grad_scale``,
        i.e. FSDP) only records the factor here; its overflow check is the finiteness of the global gradient norm,
        which :meth:`run_optimizer_step` receives (already reduced over the ranks)."""
        inv = 1.0 / self._scale
        if getattr(model, "kind", None) == "fsdp":
            model.scale_grads(inv)
            self._found_inf = None
            self._check_norm = True
            return
        self._check_norm = False
        found = torch.zeros((), device=self._gang.device)
        params = list(model.parameters())
        for p in params:
            g = p.grad
            if g is None:
                continue
            g.mul_(inv)
            found += (~torch.isfinite(g)).any().to(found.dtype)
        if self._gang.size > 1:
            self._gang.all_reduce(found, ReduceOperation.SUM)
        self._found_inf = found

    def run_optimizer_step(self, optimizer: Optimizer, *, grad_scale: Tensor | None = None,
                           grad_norm: Tensor | None = None) -> Float16LossScaleResult:
        overflow = bool(self._found_inf is not None and float(self._found_inf) > 0)
        if getattr(self, "_check_norm", False) and grad_norm is not None:
            overflow = overflow or not bool(torch.isfinite(grad_norm))
        self._found_inf = None
        old = self._scale
        if overflow:
            self._scale = max(self._scale / self._factor, 0.0)
            self._good_steps = 0
            if self._scale < self._min_scale or self._scale == 0.0:
                self._scale = max(self._min_scale, self._scale)
                return Float16LossScaleResult(old, self._scale, overflowed=True, exploded=True)
            log.info("Gradient overflow: loss scale {:g} -> {:g}; the step is skipped.", old, self._scale)
            return Float16LossScaleResult(old, self._scale, overflowed=True)
        if grad_scale is not None:
            optimizer.step(grad_scale=grad_scale)  # type: ignore[call-arg]
        else:
            optimizer.step()
        self._good_steps += 1
        if self._good_steps >= self._window:
            self._scale *= self._factor
            self._good_steps = 0
        return Float16LossScaleResult(old, self._scale)

    def get_scale(self) -> float:
        return self._scale

    def state_dict(self) -> dict[str, Any]:
        return {"scale": self._scale, "good_steps": self._good_steps}

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        self._scale = float(state_dict["scale"])
        self._good_steps = int(state_dict["good_steps"])
