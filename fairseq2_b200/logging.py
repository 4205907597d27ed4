"""``str.format`` style logger with rank-aware setup (cf. ``src/fairseq2/logging.py``)."""
from __future__ import annotations

import logging
import os
import sys
import time
from logging import DEBUG, INFO, FileHandler, Formatter, Handler, Logger, NullHandler, StreamHandler
from pathlib import Path
from typing import Any


class LogWriter:
    """Wraps a stdlib logger; messages use ``{}`` placeholders that are only
    formatted when the record is actually emitted."""

    def __init__(self, logger: str | Logger) -> None:
        self._logger = logging.getLogger(logger) if isinstance(logger, str) else logger

    def debug(self, msg: str, *args: Any, **kw: Any) -> None:
        self._write(logging.DEBUG, msg, args, kw)

    def info(self, msg: str, *args: Any, **kw: Any) -> None:
        self._write(logging.INFO, msg, args, kw)

    def warning(self, msg: str, *args: Any, **kw: Any) -> None:
        self._write(logging.WARNING, msg, args, kw)

    def error(self, msg: str, *args: Any, **kw: Any) -> None:
        self._write(logging.ERROR, msg, args, kw)

    def exception(self, msg: str, *args: Any, **kw: Any) -> None:
        kw.setdefault("exc_info", True)
        self._write(logging.ERROR, msg, args, kw)

    def _write(self, level: int, msg: str, args: tuple[Any, ...], kw: dict[str, Any]) -> None:
        if not self._logger.isEnabledFor(level):
            return
        if args:
            try:
                msg = str(msg).format(*args)
            except (IndexError, KeyError):
                msg = f"{msg} {args}"
        extra = kw.pop("extra", None)
        exc_info = kw.pop("exc_info", None)
        self._logger.log(level, msg, exc_info=exc_info, extra=extra)

    def is_enabled_for(self, level: int) -> bool:
        return self._logger.isEnabledFor(level)

    def is_enabled_for_debug(self) -> bool:
        return self._logger.isEnabledFor(DEBUG)

    def is_enabled_for_info(self) -> bool:
        return self._logger.isEnabledFor(INFO)


log = LogWriter("fairseq2_b200")


def configure_logging(*, debug: bool = False, rank: int | None = None, log_file: Path | None = None,
                      force: bool = True, no_rich: bool | None = None) -> None:
    """Console output on rank 0 only, optional per-rank file ``logs/rank_N.log``. The console handler is rich's
    (colours, wrapped tracebacks) when the stream is a terminal, unless ``no_rich`` (or ``FAIRSEQ2_NO_RICH``)."""
    if rank is None:
        rank = int(os.environ.get("RANK", "0"))
    if no_rich is None:
        no_rich = "FAIRSEQ2_NO_RICH" in os.environ
    handlers: list[Handler] = []
    if rank == 0:
        console: Handler | None = None
        if not no_rich and sys.stderr.isatty():
            try:
                from rich.logging import RichHandler

                from fairseq2_b200.utils.rich import get_error_console

                console = RichHandler(console=get_error_console(), show_path=False, keywords=[])
            except ImportError:
                console = None
        handlers.append(console if console is not None else StreamHandler(sys.stderr))
    if log_file is not None:
        log_file.parent.mkdir(parents=True, exist_ok=True)
        handlers.append(FileHandler(log_file))
    if not handlers:
        handlers.append(NullHandler())
    fmt = Formatter(f"[Rank {rank}] %(asctime)s %(levelname)s %(name)s - %(message)s")
    fmt.converter = time.gmtime
    for h in handlers:
        h.setFormatter(fmt)
    logging.basicConfig(level=DEBUG if debug else INFO, handlers=handlers, force=force)
