"""Wall-clock and device-event stopwatches (cf. ``src/fairseq2/utils/stopwatch.py``).

``Stopwatch`` keeps the reference behaviour (perf_counter, optional device
synchronize on read). ``DeviceStopwatch`` times a region with CUDA events on
the launching stream so the hot loop never needs a per-step host sync.
"""
from __future__ import annotations

from time import perf_counter
from types import TracebackType
from typing import final

import torch

from fairseq2_b200.typing import Device


@final
class Stopwatch:
    def __init__(self, *, device: Device | None = None) -> None:
        self._start: float | None = None
        self._acc = 0.0
        self._device = device if device is not None and device.type == "cuda" else None

    def start(self) -> None:
        if self._start is not None:
            raise RuntimeError("The stopwatch is already running.")
        self._sync()
        self._start = perf_counter()

    def stop(self) -> None:
        if self._start is None:
            return
        self._sync()
        self._acc += perf_counter() - self._start
        self._start = None

    def reset(self) -> None:
        self._acc = 0.0
        if self._start is not None:
            self._sync()
            self._start = perf_counter()

    def get_elapsed_time(self) -> float:
        if self._start is None:
            return self._acc
        self._sync()
        return self._acc + (perf_counter() - self._start)

    @property
    def is_running(self) -> bool:
        return self._start is not None

    def _sync(self) -> None:
        if self._device is not None:
            torch.cuda.synchronize(self._device)

    def __enter__(self) -> "Stopwatch":
        self.start()
        return self

    def __exit__(self, et: type[BaseException] | None, ev: BaseException | None, tb: TracebackType | None) -> None:
        self.stop()


@final
class DeviceStopwatch:
    """Accumulates device time of bracketed regions using CUDA events; the host
    only blocks when :meth:`get_elapsed_time` is called. Falls back to
    perf_counter on CPU."""

    def __init__(self, device: Device) -> None:
        self._cuda = device.type == "cuda"
        self._device = device
        self._pairs: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []
        self._open: torch.cuda.Event | None = None
        self._cpu = Stopwatch()

    def start(self) -> None:
        if not self._cuda:
            self._cpu.start()
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self._device))
        self._open = ev

    def stop(self) -> None:
        if not self._cuda:
            self._cpu.stop()
            return
        if self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self._device))
        self._pairs.append((self._open, ev))
        self._open = None

    def get_elapsed_time(self) -> float:
        if not self._cuda:
            return self._cpu.get_elapsed_time()
        total = 0.0
        for a, b in self._pairs:
            b.synchronize()
            total += a.elapsed_time(b) * 1e-3
        return total

    def reset(self) -> None:
        self._pairs.clear()
        self._open = None
        self._cpu.reset()
