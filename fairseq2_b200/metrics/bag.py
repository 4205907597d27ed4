"""A named collection of metrics with transactional updates and one-shot
synchronisation (cf. fairseq2 ``metrics/bag.py:26-145``).

``begin_updates``/``commit_updates``/``rollback_updates`` let the trainer drop
the metric updates of a step that is retried after an fp16 overflow.
``sync_and_compute_metrics`` packs all metric states into one fp64 vector per
reduction kind and all-reduces it once."""
from __future__ import annotations

from copy import deepcopy
from typing import Any, Iterable, Mapping, Sequence

import torch
from torch import Tensor

from fairseq2_b200.gang import Gang, ReduceOperation
from fairseq2_b200.metrics.aggregation import Metric
from fairseq2_b200.typing import Device


class MetricBag:
    def __init__(self, device: Device) -> None:
        self.device = device
        self._metrics: dict[str, Metric] = {}
        self._backup: dict[str, Tensor] | None = None

    def add(self, name: str, metric: Metric) -> Metric:
        if name in self._metrics:
            raise ValueError(f"The bag already has a metric named '{name}'.")
        self._metrics[name] = metric.to(self.device)
        return metric

    def get(self, name: str, kls: type[Metric] | None = None) -> Metric:
        m = self._metrics.get(name)
        if m is None:
            if kls is None:
                raise KeyError(f"The bag does not have a metric named '{name}'.")
            m = self.add(name, kls(self.device))
        elif kls is not None and not isinstance(m, kls):
            raise TypeError(f"The metric '{name}' is of type `{type(m).__name__}`, not `{kls.__name__}`.")
        return m

    def __contains__(self, name: str) -> bool:
        return name in self._metrics

    @property
    def metrics(self) -> Mapping[str, Metric]:
        return self._metrics

    def begin_updates(self) -> None:
        if self._backup is not None:
            raise ValueError("`begin_updates()` has already been called.")
        self._backup = {n: m.state.clone() for n, m in self._metrics.items()}

    def commit_updates(self) -> None:
        if self._backup is None:
            raise ValueError("`begin_updates()` must be called first.")
        self._backup = None

    def rollback_updates(self) -> None:
        if self._backup is None:
            raise ValueError("`begin_updates()` must be called first.")
        for n in list(self._metrics):
            if n in self._backup:
                self._metrics[n].state = self._backup[n]
            else:
                del self._metrics[n]
        self._backup = None

    def reset_metrics(self) -> None:
        for m in self._metrics.values():
            m.reset()

    def reset_non_persistent_metrics(self) -> None:
        for n, m in self._metrics.items():
            if not n.startswith("total_"):
                m.reset()

    def state_dict(self) -> dict[str, Any]:
        return {n: m.state_dict() for n, m in self._metrics.items() if n.startswith("total_")}

    def load_state_dict(self, sd: Mapping[str, Any]) -> None:
        for n, s in sd.items():
            if n in self._metrics:
                self._metrics[n].load_state_dict(s)


def sync_and_compute_metrics(bag: MetricBag | Sequence[MetricBag], gang: Gang | None = None
                             ) -> dict[str, Any] | None:
    """All ranks call; rank 0 gets ``{name: python scalar}``, others ``None``."""
    bags = [bag] if isinstance(bag, MetricBag) else list(bag)
    items: list[tuple[str, Metric]] = []
    for b in bags:
        items.extend(b.metrics.items())
    if not items:
        return {} if gang is None or gang.rank == 0 else None
    states = {n: m.state.clone() for n, m in items}
    if gang is not None and gang.size > 1:
        for op in (ReduceOperation.SUM, ReduceOperation.MAX, ReduceOperation.MIN):
            group = [(n, m) for n, m in items if m.reduce_op == op]
            if not group:
                continue
            packed = torch.cat([states[n].to(gang.device) for n, _ in group])
            gang.all_reduce(packed, op)
            off = 0
            for n, m in group:
                states[n] = packed[off: off + m.state_size]
                off += m.state_size
    if gang is not None and gang.rank != 0:
        return None
    names = [n for n, _ in items]
    outs = [m.compute_from(states[n]).to(torch.float64).reshape(-1) for n, m in items]
    flat = torch.cat([o.to(outs[0].device) for o in outs]).cpu().tolist()  # one D2H
    result: dict[str, Any] = {}
    off = 0
    for n, o in zip(names, outs):
        k = o.numel()
        result[n] = flat[off] if k == 1 else flat[off: off + k]   # multi-valued metrics (e.g. UER + WER) stay lists
        off += k
    return result
