"""Bag of random number generators with save/restore (cf. ``src/fairseq2/utils/rng.py``)."""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Iterator, Mapping, Sequence

import torch
from torch import Generator

from fairseq2_b200.typing import Device


class RngBag:
    """Holds the default generators of a set of devices (CPU is always present
    when built via :meth:`from_device_defaults`)."""

    def __init__(self, *generators: Generator) -> None:
        self._generators = list(generators)

    @staticmethod
    def from_device_defaults(*devices: Device) -> "RngBag":
        seen: set[str] = set()
        gens: list[Generator] = []
        for d in devices:
            key = str(d)
            if key in seen:
                raise ValueError(f"`devices` must be unique, but '{key}' is given more than once.")
            seen.add(key)
            if d.type == "cpu":
                gens.append(torch.default_generator)
            elif d.type == "cuda":
                idx = d.index if d.index is not None else torch.cuda.current_device()
                torch.cuda.init()
                gens.append(torch.cuda.default_generators[idx])
            else:
                raise ValueError(f"`devices` must be of type cpu or cuda, but '{key}' is given.")
        return RngBag(*gens)

    def seed(self) -> None:
        if self._generators:
            self._generators[0].seed()
            s = self._generators[0].initial_seed()
            for g in self._generators[1:]:
                g.manual_seed(s)

    def manual_seed(self, seed: int) -> None:
        if seed < 0 or seed >= 1 << 32:
            raise ValueError(f"`seed` must be in [0, 2^32), but is {seed} instead.")
        for g in self._generators:
            g.manual_seed(seed)

    @contextmanager
    def temporary_manual_seed(self, seed: int) -> Iterator[None]:
        saved = [g.get_state() for g in self._generators]
        self.manual_seed(seed)
        try:
            yield
        finally:
            for g, s in zip(self._generators, saved):
                g.set_state(s)

    def state_dict(self) -> dict[str, Any]:
        return {"generators": [g.get_state() for g in self._generators]}

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        states = state_dict.get("generators")
        if not isinstance(states, Sequence) or len(states) != len(self._generators):
            raise ValueError(
                f"`state_dict['generators']` must hold {len(self._generators)} generator state(s).")
        for g, s in zip(self._generators, states):
            g.set_state(s.cpu() if isinstance(s, torch.Tensor) else s)


@contextmanager
def temporary_manual_seed(seed: int, *devices: Device) -> Iterator[None]:
    with RngBag.from_device_defaults(*devices).temporary_manual_seed(seed):
        yield
