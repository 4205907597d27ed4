"""rich-backed console and progress reporting (fairseq2 ``utils/rich.py:34-149``).

A process-wide console pair (stdout / stderr) that logging and the CLI share, and ``RichProgressReporter``, a
``ProgressReporter`` whose tasks render as bars with an ``n/N`` column, elapsed time and ETA on the error console.
"""

from __future__ import annotations

from types import TracebackType

from rich.console import Console
from rich.progress import BarColumn, Progress, ProgressColumn, Task, TaskID, TextColumn, TimeElapsedColumn, TimeRemainingColumn
from rich.text import Text

from fairseq2_b200.utils.progress import ProgressReporter, ProgressTask

_console: Console | None = None
_error_console: Console | None = None


def get_console() -> Console:
    global _console
    if _console is None:
        _console = Console(highlight=False)
    return _console


def set_console(console: Console) -> None:
    global _console
    _console = console


def get_error_console() -> Console:
    global _error_console
    if _error_console is None:
        _error_console = Console(stderr=True, highlight=False)
    return _error_console


def set_error_console(console: Console) -> None:
    global _error_console
    _error_console = console


class BasicMofNCompleteColumn(ProgressColumn):
    """``completed/total`` when the total is known, otherwise just ``completed``."""

    def render(self, task: Task) -> Text:
        done = int(task.completed)
        if task.total is None:
            return Text(f"{done:5d}", style="progress.download")
        total = int(task.total)
        width = len(str(total))
        return Text(f"{done:{width}d}/{total}", style="progress.download")


def _columns() -> list[ProgressColumn]:
    return [TextColumn("{task.description}:"), BarColumn(), BasicMofNCompleteColumn(), TimeElapsedColumn(),
            TimeRemainingColumn()]


class RichProgressTask(ProgressTask):
    def __init__(self, progress: Progress, task_id: TaskID) -> None:
        self._progress = progress
        self._task_id = task_id

    def start(self) -> None:
        self._progress.start_task(self._task_id)

    def step(self, n: int = 1) -> None:
        self._progress.update(self._task_id, advance=n)

    def close(self) -> None:
        self._progress.remove_task(self._task_id)


class RichProgressReporter(ProgressReporter):
    """Use as a context manager around the loop whose tasks should be drawn; outside it tasks are silent."""

    def __init__(self, console: Console | None = None, transient: bool = True) -> None:
        self._progress = Progress(*_columns(), console=console or get_error_console(), transient=transient)

    def create_task(self, name: str, total: int | None, completed: int = 0, *, start: bool = True) -> ProgressTask:
        task_id = self._progress.add_task(name, start=start, total=total, completed=completed)
        return RichProgressTask(self._progress, task_id)

    def __enter__(self) -> "RichProgressReporter":
        self._progress.start()
        return self

    def __exit__(self, et: type[BaseException] | None, ev: BaseException | None, tb: TracebackType | None) -> None:
        self._progress.stop()
