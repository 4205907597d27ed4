"""Small structural types shared across the package (cf. ``src/fairseq2/typing.py``)."""
from __future__ import annotations

from contextlib import AbstractContextManager
from typing import Any, Mapping, Protocol, TypeAlias, TypeVar, runtime_checkable

import torch

T = TypeVar("T")

ContextManager: TypeAlias = AbstractContextManager[None]
Device: TypeAlias = torch.device
DataType: TypeAlias = torch.dtype


@runtime_checkable
class Stateful(Protocol):
    """An object whose state can be captured and restored."""

    def state_dict(self) -> dict[str, Any]: ...

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None: ...


class Closable(Protocol):
    def close(self) -> None: ...


def safe_cast(name: str, value: object, kls: type[T]) -> T:
    if not isinstance(value, kls):
        raise TypeError(f"`{name}` must be of type `{kls}`, but is of type `{type(value)}` instead.")
    return value
