"""A value built on first use (cf. fairseq2 ``runtime/lazy.py:15-29``)."""
from __future__ import annotations

import threading
from typing import Callable, Generic, TypeVar

T_co = TypeVar("T_co", covariant=True)

_UNSET = object()


class Lazy(Generic[T_co]):
    """``Lazy(factory).get()`` calls ``factory`` once, also under concurrent first calls, and drops it afterwards."""

    def __init__(self, factory: Callable[[], T_co]) -> None:
        self._factory: Callable[[], T_co] | None = factory
        self._value: object = _UNSET
        self._lock = threading.Lock()

    def get(self) -> T_co:
        if self._value is _UNSET:
            with self._lock:
                if self._value is _UNSET:
                    assert self._factory is not None
                    self._value = self._factory()
                    self._factory = None
        return self._value  # type: ignore[return-value]
