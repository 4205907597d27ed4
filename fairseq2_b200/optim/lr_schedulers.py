"""Learning-rate schedulers (cf. fairseq2 ``optim/lr_schedulers/*``):
cosine annealing with warm restarts, Myle, Noam, polynomial decay, tri-stage
and passthrough. All are ``torch.optim.lr_scheduler.LRScheduler`` subclasses
that compute a closed-form LR from ``last_epoch`` (= number of ``step()``
calls) for every parameter group."""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Sequence

from torch.optim import Optimizer
from torch.optim.lr_scheduler import LRScheduler


class AbstractLRScheduler(ABC, LRScheduler):
    def get_lr(self) -> list[float]:  # type: ignore[override]
        return self._compute_lrs()

    @abstractmethod
    def _compute_lrs(self) -> list[float]: ...


def _per_group(value: float | Sequence[float], optimizer: Optimizer, name: str) -> list[float]:
    n = len(optimizer.param_groups)
    if isinstance(value, (int, float)):
        return [float(value)] * n
    v = list(value)
    if len(v) != n:
        raise ValueError(f"The length of `{name}` must equal the number of parameter groups ({n}), but is {len(v)}.")
    return [float(x) for x in v]


class PassthroughLR(AbstractLRScheduler):
    """Keeps the base learning rates."""

    def __init__(self, optimizer: Optimizer, *, last_epoch: int = -1) -> None:
        super().__init__(optimizer, last_epoch)

    def _compute_lrs(self) -> list[float]:
        return list(self.base_lrs)


NoopLR = PassthroughLR


class CosineAnnealingLR(AbstractLRScheduler):
    """Linear warm-up from ``start_lr`` then cosine cycles; cycle ``k`` has
    length ``cycle_len * cycle_mul**k`` and its min/max LRs are scaled by
    ``lr_mul**k`` (SGDR)."""

    def __init__(self, optimizer: Optimizer, cycle_len: int, num_warmup_steps: int, *, cycle_mul: float = 1.0,
                 lr_mul: float = 1.0, start_lr: float | Sequence[float] = 0.0,
                 final_lr: float | Sequence[float] = 0.0, last_epoch: int = -1) -> None:
        if cycle_len <= 0:
            raise ValueError(f"`cycle_len` must be positive, but is {cycle_len} instead.")
        self._cycle_len, self._cycle_mul, self._warmup, self._lr_mul = cycle_len, cycle_mul, num_warmup_steps, lr_mul
        self._start_lrs = _per_group(start_lr, optimizer, "start_lr")
        self._final_lrs = _per_group(final_lr, optimizer, "final_lr")
        super().__init__(optimizer, last_epoch)

    def _compute_lrs(self) -> list[float]:
        t = self.last_epoch
        base = self.base_lrs
        if t < self._warmup:
            c = t / self._warmup
            return [s + (b - s) * c for s, b in zip(self._start_lrs, base)]
        cur = t - self._warmup
        if self._cycle_mul == 1.0:
            k = cur // self._cycle_len
            length = self._cycle_len
            pos = cur - k * self._cycle_len
        else:
            i = math.floor(math.log(1 - cur / self._cycle_len * (1 - self._cycle_mul), self._cycle_mul))
            k = i
            length = self._cycle_len * self._cycle_mul ** i
            start = (1 - self._cycle_mul ** i) / (1 - self._cycle_mul) * self._cycle_len
            pos = cur - start
        m = self._lr_mul ** k
        c = math.cos(math.pi * pos / length)
        return [f * m + 0.5 * (b * m - f * m) * (1 + c) for b, f in zip(base, self._final_lrs)]


class MyleLR(AbstractLRScheduler):
    """Linear warm-up, then ``base * sqrt(warmup / t)``."""

    def __init__(self, optimizer: Optimizer, num_warmup_steps: int, *, start_lr: float | Sequence[float] = 0.0,
                 last_epoch: int = -1) -> None:
        if num_warmup_steps == 0:
            raise ValueError("`num_warmup_steps` must be greater than 0.")
        self._warmup = num_warmup_steps
        self._start_lrs = _per_group(start_lr, optimizer, "start_lr")
        super().__init__(optimizer, last_epoch)

    def _compute_lrs(self) -> list[float]:
        t = self.last_epoch
        if t < self._warmup:
            c = t / self._warmup
            return [s + (b - s) * c for s, b in zip(self._start_lrs, self.base_lrs)]
        c = (self._warmup / t) ** 0.5
        return [b * c for b in self.base_lrs]


class NoamLR(AbstractLRScheduler):
    """``base * min(t * warmup^-1.5, t^-0.5)`` (Vaswani et al.)."""

    def __init__(self, optimizer: Optimizer, num_warmup_steps: int, *, last_epoch: int = -1) -> None:
        self._warmup = num_warmup_steps
        super().__init__(optimizer, last_epoch)

    def _compute_lrs(self) -> list[float]:
        t = self.last_epoch
        if t == 0:
            return [0.0] * len(self.base_lrs)
        c = min(t ** -0.5, t * self._warmup ** -1.5) if self._warmup > 0 else t ** -0.5
        return [b * c for b in self.base_lrs]


class PolynomialDecayLR(AbstractLRScheduler):
    """Warm-up, then ``final + (base - final) * ((N - t) / (N - W))**power``; ``final`` after ``N``."""

    def __init__(self, optimizer: Optimizer, num_steps: int, num_warmup_steps: int, *, power: float = 1.0,
                 start_lr: float | Sequence[float] = 0.0, final_lr: float | Sequence[float] = 0.0,
                 last_epoch: int = -1) -> None:
        if num_warmup_steps >= num_steps:
            raise ValueError(f"`num_warmup_steps` must be less than `num_steps` ({num_steps}), but is {num_warmup_steps}.")
        self._num_steps, self._warmup, self._power = num_steps, num_warmup_steps, power
        self._start_lrs = _per_group(start_lr, optimizer, "start_lr")
        self._final_lrs = _per_group(final_lr, optimizer, "final_lr")
        super().__init__(optimizer, last_epoch)

    def _compute_lrs(self) -> list[float]:
        t = self.last_epoch
        if t < self._warmup:
            c = t / self._warmup
            return [s + (b - s) * c for s, b in zip(self._start_lrs, self.base_lrs)]
        if t >= self._num_steps:
            return list(self._final_lrs)
        c = ((self._num_steps - t) / (self._num_steps - self._warmup)) ** self._power
        return [f + (b - f) * c for b, f in zip(self.base_lrs, self._final_lrs)]


class TriStageLR(AbstractLRScheduler):
    """Warm-up from ``start_lr_scale * base``, hold at ``base``, exponential
    decay to ``final_lr_scale * base``; stage lengths are ``stage_ratio * num_steps``."""

    def __init__(self, optimizer: Optimizer, num_steps: int, stage_ratio: tuple[float, float, float], *,
                 start_lr_scale: float | Sequence[float] = 0.01, final_lr_scale: float | Sequence[float] = 0.01,
                 last_epoch: int = -1) -> None:
        if not math.isclose(sum(stage_ratio), 1.0, rel_tol=1e-6):
            raise ValueError(f"The sum of `stage_ratio` must be 1.0, but is {sum(stage_ratio)} instead.")
        self._num_steps = num_steps
        self._s1 = int(num_steps * stage_ratio[0])
        self._s2 = int(num_steps * stage_ratio[1])
        self._s3 = int(num_steps * stage_ratio[2])
        self._start_scales = _per_group(start_lr_scale, optimizer, "start_lr_scale")
        self._final_scales = _per_group(final_lr_scale, optimizer, "final_lr_scale")
        super().__init__(optimizer, last_epoch)

    def _compute_lrs(self) -> list[float]:
        t = self.last_epoch
        base = self.base_lrs
        if t < self._s1:
            c = t / self._s1
            return [b * s + (b - b * s) * c for b, s in zip(base, self._start_scales)]
        t -= self._s1
        if t < self._s2:
            return list(base)
        t -= self._s2
        if t < self._s3:
            c = t / self._s3
            return [b * math.exp(math.log(f) * c) for b, f in zip(base, self._final_scales)]
        return [b * f for b, f in zip(base, self._final_scales)]


def get_effective_lr(scheduler: LRScheduler) -> float:
    return float(scheduler.get_last_lr()[0])
