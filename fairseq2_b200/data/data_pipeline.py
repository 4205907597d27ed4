"""Python face of the native data pipeline (cf. fairseq2 ``data/data_pipeline.py:19-717``).

Everything that touches examples -- sources, operators, the collater, file
mapping, text parsing, audio/image decoding -- is implemented in C++ in
``csrc/data`` and runs without the GIL except while a Python callback executes.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path
from typing import Any, TypedDict

from torch import Tensor

_PKG = Path(__file__).resolve().parent.parent


def _load_native():  # type: ignore[no-untyped-def]
    import torch  # noqa: F401

    path = _PKG / "_data.so"
    if not path.exists():
        raise ImportError(f"The native data runtime '{path}' has not been built. Run `python -m fairseq2_b200.csrc.build`.")
    name = "fairseq2_b200._data"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    assert spec is not None and spec.loader is not None
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_n = _load_native()

DataPipeline = _n.DataPipeline
DataPipelineBuilder = _n.DataPipelineBuilder
DataPipelineError = _n.DataPipelineError
ByteStreamError = _n.ByteStreamError
RecordError = _n.RecordError
Collater = _n.Collater
CollateOptionsOverride = _n.CollateOptionsOverride
FileMapper = _n.FileMapper
MemoryBlock = _n.MemoryBlock
list_files = _n.list_files
read_sequence = _n.read_sequence
read_zipped_records = _n.read_zipped_records
read_iterator = _n.read_iterator


class FileMapperOutput(TypedDict):
    """What a :class:`FileMapper` returns for one pathname: the path relative to
    the mapper's root and the bytes of the file, or of the requested slice of it
    (cf. fairseq2 ``data/data_pipeline.py``, ``FileMapperOutput``)."""

    path: str
    data: "MemoryBlock"


class SequenceData(TypedDict):
    """Output of the collater for padded sequences."""

    seqs: Tensor
    seq_lens: list[int]
    is_ragged: bool


def get_last_failed_example() -> Any:
    """Kept for API compatibility; the native runtime reports the failing
    example inside the raised ``DataPipelineError`` message instead."""
    return None


def create_bucket_sizes(*, max_num_elements: int, max_seq_len: int, min_seq_len: int = 1,
                        num_seqs_multiple_of: int = 1) -> list[tuple[int, int]]:
    """Bucket table ``[(batch_size, seq_len)]`` for ``bucket_by_length`` such
    that ``batch_size * seq_len <= max_num_elements`` and ``batch_size`` is a
    multiple of ``num_seqs_multiple_of`` (cf. reference ``data_pipeline.py:646-717``)."""
    if max_seq_len > max_num_elements:
        raise ValueError(f"`max_seq_len` must be less than or equal to `max_num_elements` ({max_num_elements}), but is {max_seq_len} instead.")
    if min_seq_len < 1:
        raise ValueError(f"`min_seq_len` must be greater than zero, but is {min_seq_len} instead.")
    if min_seq_len > max_seq_len:
        raise ValueError(f"`min_seq_len` must be less than or equal to `max_seq_len` ({max_seq_len}), but is {min_seq_len} instead.")
    if num_seqs_multiple_of < 1:
        raise ValueError(f"`num_seqs_multiple_of` must be greater than or equal to 1, but is {num_seqs_multiple_of} instead.")
    if max_num_elements % max_seq_len != 0:
        raise ValueError(f"`max_num_elements` must be equal to a multiple of `max_seq_len`, but is {max_num_elements} instead.")
    if max_num_elements < max_seq_len * num_seqs_multiple_of:
        raise ValueError("`max_num_elements` must be greater than or equal to `max_seq_len * num_seqs_multiple_of`.")
    # One entry per distinct value of `max_num_elements // seq_len`, at the longest `seq_len` that still allows that
    # many rows; the row count is then rounded down to the multiple (so two entries may share a row count).
    sizes: list[tuple[int, int]] = []
    seq_len = min_seq_len
    while seq_len <= max_seq_len:
        rows = max_num_elements // seq_len
        last = min(max_num_elements // rows, max_seq_len)          # longest length with the same number of rows
        rounded = rows - rows % num_seqs_multiple_of
        if rounded > 0:
            sizes.append((rounded, last))
        seq_len = last + 1
    return sizes
