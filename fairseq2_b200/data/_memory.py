"""Module path of :class:`MemoryBlock` that existing code imports from
(cf. fairseq2 ``data/_memory.py``). The class itself is the native one: a
reference-counted, read-only view over bytes owned by C++ (an mmap'd file, a
heap buffer, a Python buffer object) that exports the buffer protocol."""
from __future__ import annotations

from typing import TypeAlias, Union

from fairseq2_b200.data.data_pipeline import MemoryBlock

Buffer: TypeAlias = Union[bytes, bytearray, memoryview, "array.array"]  # noqa: F821

__all__ = ["Buffer", "MemoryBlock"]
