"""Python GC control for training loops (cf. ``src/fairseq2/utils/gc.py``):
automatic collection is switched off and a generation-1 collection runs every
N steps so that all ranks pause at the same step instead of at random ones."""
from __future__ import annotations

import gc
from types import TracebackType


class GarbageCollector:
    def enable(self, value: bool = True) -> None: ...

    def step(self) -> None: ...


class NoopGarbageCollector(GarbageCollector):
    pass


class CPythonGarbageCollector(GarbageCollector):
    def __init__(self, collect_every_n_step: int) -> None:
        if collect_every_n_step <= 0:
            raise ValueError("`collect_every_n_step` must be positive.")
        self._n = collect_every_n_step
        self._step = 0
        self._enabled = False

    def enable(self, value: bool = True) -> None:
        self._enabled = value
        self._step = 0
        if value:
            gc.disable()
        else:
            gc.enable()

    def step(self) -> None:
        if not self._enabled:
            return
        self._step += 1
        if self._step % self._n == 0:
            gc.collect(generation=1)

    def __enter__(self) -> "CPythonGarbageCollector":
        self.enable(True)
        return self

    def __exit__(self, et: type[BaseException] | None, ev: BaseException | None, tb: TracebackType | None) -> None:
        self.enable(False)
