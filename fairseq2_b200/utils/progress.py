"""Progress reporting abstraction (cf. ``src/fairseq2/utils/progress.py``). A
``tqdm`` backend is used when stderr is a TTY and ``FAIRSEQ2_NO_PROGRESS`` is
unset; otherwise reporting is a no-op."""
from __future__ import annotations

import os
import sys
from types import TracebackType


class ProgressTask:
    def step(self, n: int = 1) -> None: ...

    def close(self) -> None: ...

    def __enter__(self) -> "ProgressTask":
        return self

    def __exit__(self, et: type[BaseException] | None, ev: BaseException | None, tb: TracebackType | None) -> None:
        self.close()


class ProgressReporter:
    def create_task(self, name: str, total: int | None, completed: int = 0) -> ProgressTask:
        return ProgressTask()


class _TqdmTask(ProgressTask):
    def __init__(self, name: str, total: int | None, completed: int) -> None:
        from tqdm import tqdm

        self._bar = tqdm(total=total, initial=completed, desc=name, file=sys.stderr, leave=False)

    def step(self, n: int = 1) -> None:
        self._bar.update(n)

    def close(self) -> None:
        self._bar.close()


class TqdmProgressReporter(ProgressReporter):
    def create_task(self, name: str, total: int | None, completed: int = 0) -> ProgressTask:
        return _TqdmTask(name, total, completed)


def create_progress_reporter(rank: int = 0) -> ProgressReporter:
    if rank != 0 or os.environ.get("FAIRSEQ2_NO_PROGRESS") or not sys.stderr.isatty():
        return ProgressReporter()
    return TqdmProgressReporter()
