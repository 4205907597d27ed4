"""Current default floating-point dtype as a context (cf. ``src/fairseq2/data_type.py``)."""
from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Iterator

import torch

from fairseq2_b200.typing import DataType

_tls = threading.local()


def get_current_dtype() -> DataType:
    stack = getattr(_tls, "stack", None)
    if stack:
        return stack[-1]
    return torch.get_default_dtype()


def get_default_dtype() -> DataType:
    return torch.get_default_dtype()


@contextmanager
def set_dtype(dtype: DataType) -> Iterator[None]:
    """Makes ``dtype`` the default floating dtype of torch factory functions
    inside the block (module constructors pick it up)."""
    stack = getattr(_tls, "stack", None)
    if stack is None:
        stack = _tls.stack = []
    prev = torch.get_default_dtype()
    stack.append(dtype)
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(prev)
        stack.pop()


default_dtype = set_dtype
