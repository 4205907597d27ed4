"""Third-party extensions: functions ``extension(container)`` published under an entry-point group.

Behaviour follows the reference (``fairseq2/composition/extensions.py:17-52``): every entry point of the group is
loaded and called with the container; a failing extension is logged and skipped unless ``FAIRSEQ2_EXTENSION_TRACE`` is
set, in which case the failure is raised as ``ExtensionError`` with the original exception as its cause.
"""

from __future__ import annotations

import inspect
import os
from importlib.metadata import entry_points
from typing import Any, Iterable

from fairseq2_b200.logging import log
from fairseq2_b200.runtime.dependency import DependencyContainer

EXTENSION_GROUP = "fairseq2_b200.extension"


class ExtensionError(Exception):
    def __init__(self, entry_point: str, message: str) -> None:
        super().__init__(message)
        self.entry_point = entry_point


def _accepts_container(fn: Any) -> bool:
    """True if ``fn`` can be called with exactly one positional argument."""
    try:
        sig = inspect.signature(fn)
    except (TypeError, ValueError):
        return True                      # builtins and the like: let the call decide
    try:
        sig.bind(object())
    except TypeError:
        return False
    return True


def run_extensions(container: DependencyContainer, *, group: str = EXTENSION_GROUP,
                   points: Iterable[Any] | None = None) -> list[str]:
    """Calls every extension of ``group`` with ``container``; returns the names of those that ran.

    ``points`` replaces the entry-point lookup (objects with ``value``, ``load()``), which is how tests inject fakes.
    """
    trace = "FAIRSEQ2_EXTENSION_TRACE" in os.environ
    if points is None:
        points = entry_points(group=group)
    ran: list[str] = []
    for ep in points:
        name = getattr(ep, "value", str(ep))
        try:
            fn = ep.load()
            if not _accepts_container(fn):
                msg = (f"{name} entry point cannot be run as an extension since its signature does not match "
                       "`extension_function(container: DependencyContainer)`.")
                if trace:
                    raise ExtensionError(name, msg)
                log.warning("%s Set `FAIRSEQ2_EXTENSION_TRACE` to raise instead.", msg)
                continue
            fn(container)
        except ExtensionError:
            raise
        except Exception as ex:  # noqa: BLE001 - an extension is foreign code; one bad package must not break start-up
            if trace:
                raise ExtensionError(name, f"{name} extension failed.") from ex
            log.warning("%s extension failed (%s: %s). Set `FAIRSEQ2_EXTENSION_TRACE` to raise instead.", name,
                        type(ex).__name__, ex)
            continue
        ran.append(name)
        if trace:
            log.info("%s extension registered successfully.", name)
    return ran
