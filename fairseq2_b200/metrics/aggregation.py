"""Streaming aggregations kept on the device (cf. fairseq2 ``metrics/aggregation.py``).

State is a small fp64 vector so that every metric of a bag can be synchronised
across ranks with ONE packed all-reduce (see ``MetricBag.sync``) instead of a
pickled ``all_gather_object`` per publish."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Mapping

import torch
from torch import Tensor

from fairseq2_b200.gang import ReduceOperation
from fairseq2_b200.typing import Device


class Metric(ABC):
    #: how ``state`` combines across ranks
    reduce_op: ReduceOperation = ReduceOperation.SUM
    state_size: int = 1

    def __init__(self, device: Device | None = None) -> None:
        self.device = device or torch.device("cpu")
        self.state = self._initial()

    def _initial(self) -> Tensor:
        return torch.zeros(self.state_size, dtype=torch.float64, device=self.device)

    def reset(self) -> None:
        self.state = self._initial()

    def to(self, device: Device) -> "Metric":
        self.device = device
        self.state = self.state.to(device)
        return self

    @abstractmethod
    def update(self, value: Any, **kw: Any) -> None: ...

    @abstractmethod
    def compute_from(self, state: Tensor) -> Tensor: ...

    def compute(self) -> Tensor:
        return self.compute_from(self.state)

    def state_dict(self) -> dict[str, Any]:
        return {"state": self.state.detach().cpu()}

    def load_state_dict(self, sd: Mapping[str, Any]) -> None:
        self.state = sd["state"].to(self.device, torch.float64)


def _as64(v: Any, device: Device) -> Tensor:
    if isinstance(v, Tensor):
        return v.detach().to(device=device, dtype=torch.float64)
    return torch.tensor(float(v), dtype=torch.float64, device=device)


class Sum(Metric):
    def update(self, value: Any, *, weight: float = 1.0) -> None:
        self.state = self.state + _as64(value, self.device).sum() * weight

    def compute_from(self, state: Tensor) -> Tensor:
        return state[0]


class Mean(Metric):
    """Weighted mean: ``sum(value * weight) / sum(weight)``."""

    state_size = 2

    def update(self, value: Any, *, weight: Any = 1.0) -> None:
        v, w = _as64(value, self.device), _as64(weight, self.device)
        self.state = self.state + torch.stack([(v * w).sum(), w.sum() if w.ndim else w * max(v.numel(), 1)])

    def compute_from(self, state: Tensor) -> Tensor:
        return state[0] / state[1].clamp(min=1e-300)


class Max(Metric):
    reduce_op = ReduceOperation.MAX

    def _initial(self) -> Tensor:
        return torch.full((1,), float("-inf"), dtype=torch.float64, device=self.device)

    def update(self, value: Any) -> None:
        self.state = torch.maximum(self.state, _as64(value, self.device).max().reshape(1))

    def compute_from(self, state: Tensor) -> Tensor:
        return state[0]


class Min(Metric):
    reduce_op = ReduceOperation.MIN

    def _initial(self) -> Tensor:
        return torch.full((1,), float("inf"), dtype=torch.float64, device=self.device)

    def update(self, value: Any) -> None:
        self.state = torch.minimum(self.state, _as64(value, self.device).min().reshape(1))

    def compute_from(self, state: Tensor) -> Tensor:
        return state[0]
