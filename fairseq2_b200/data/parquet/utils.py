"""Arrow <-> torch conversion and small Arrow helpers used by the Parquet stages
(fairseq2 ``data/parquet/utils.py:30-256``)."""

from __future__ import annotations

import os
import uuid
import weakref
import zlib
from collections.abc import Iterator
from contextlib import contextmanager
from pathlib import Path
from typing import Any, Union

import numpy as np
import pyarrow as pa
import pyarrow.dataset as ds
import pyarrow.parquet as pq
import torch
from torch import Tensor

NestedDictValue = Union[Tensor, list[Any], "pa.Array", dict[str, Any]]
NestedDict = dict[str, NestedDictValue]
BatchOutputType = Union[pa.Table, NestedDict]


def circular_shift_left(items: list[Any], k: int) -> list[Any]:
    if len(items) <= 1:
        return items
    k %= len(items)
    return items[k:] + items[:k]


def fragment_stable_hash(fragment: ds.Fragment, seed: int | None = None) -> int:
    """Hash of (file path, row-group ids, seed) that is the same in every process and run (``hash()`` is not)."""
    key = f"{fragment.path}-{[rg.id for rg in fragment.row_groups]}-{seed}"
    return zlib.crc32(key.encode("utf-8"))


def pyarrow_column_to_array(arr: pa.Array | pa.ChunkedArray) -> pa.Array:
    if isinstance(arr, pa.ChunkedArray):
        return arr.chunk(0) if arr.num_chunks == 1 else arr.combine_chunks()
    return arr


def _numpy_or_none(arr: pa.Array) -> np.ndarray | None:
    try:
        return arr.to_numpy(zero_copy_only=True)
    except (pa.ArrowInvalid, pa.ArrowNotImplementedError, NotImplementedError):
        return None


def pyarrow_to_torch_tensor(arr: pa.Array | pa.ChunkedArray, strict: bool = False) -> NestedDictValue:
    """Best-effort conversion of one column: numeric -> tensor (zero copy when possible), strings -> ``list[str]``,
    list<numeric> -> list of 1-D tensors, list<fixed_size_list<numeric>> -> list of 2-D tensors,
    fixed_size_list<numeric> -> 2-D tensor, struct -> dict, dictionary -> decoded. Nulls are rejected."""
    if arr.null_count != 0:
        raise ValueError("Conversion to torch does not support null values.")
    arr = pyarrow_column_to_array(arr)
    t = arr.type
    np_view = _numpy_or_none(arr)
    if np_view is not None and np_view.dtype != object:
        return torch.from_numpy(np_view)
    if pa.types.is_boolean(t):
        return torch.from_numpy(arr.to_numpy(zero_copy_only=False))
    if pa.types.is_dictionary(t):
        return pyarrow_to_torch_tensor(arr.dictionary_decode(), strict)
    if pa.types.is_string(t) or pa.types.is_large_string(t):
        return arr.to_pylist()
    if pa.types.is_list(t) or pa.types.is_large_list(t):
        vt = t.value_type
        offsets = arr.offsets.to_numpy()
        if pa.types.is_primitive(vt):
            flat = torch.from_numpy(np.asarray(arr.values.to_numpy(zero_copy_only=False)))
            return [flat[offsets[i]: offsets[i + 1]] for i in range(len(arr))]
        if pa.types.is_fixed_size_list(vt) and pa.types.is_primitive(vt.value_type):
            inner = np.asarray(arr.values.values.to_numpy(zero_copy_only=False)).reshape(-1, vt.list_size)
            flat = torch.from_numpy(inner)
            return [flat[offsets[i]: offsets[i + 1]] for i in range(len(arr))]
    if pa.types.is_fixed_size_list(t) and pa.types.is_primitive(t.value_type):
        n = len(arr)
        values = arr.values.to_numpy(zero_copy_only=False)[arr.offset * t.list_size: (arr.offset + n) * t.list_size]
        return torch.from_numpy(np.asarray(values).reshape(n, t.list_size))
    if pa.types.is_struct(t):
        return {t.field(i).name: pyarrow_to_torch_tensor(arr.field(i), strict) for i in range(t.num_fields)}
    if pa.types.is_nested(t):
        raise NotImplementedError(f"Nested type {t} is not supported.")
    if strict:
        raise NotImplementedError(f"{t} cannot be converted to a torch.Tensor.")
    return arr


def pyarrow_table_to_torch_dict(table: pa.Table, strict: bool = False) -> NestedDict:
    """Column name -> converted column; a column that cannot be converted stays an Arrow array unless ``strict``."""
    out: NestedDict = {}
    for name in table.column_names:
        try:
            out[name] = pyarrow_to_torch_tensor(table[name], strict)
        except ValueError:
            if strict:
                raise
            out[name] = table[name]
    return out


@contextmanager
def pyarrow_cpu(nb_cpu: int) -> Iterator[None]:
    """Temporarily sets Arrow's compute and IO thread pools to ``nb_cpu`` threads."""
    cpu, io = pa.cpu_count(), pa.io_thread_count()
    pa.set_cpu_count(nb_cpu)
    pa.set_io_thread_count(nb_cpu)
    try:
        yield
    finally:
        pa.set_cpu_count(cpu)
        pa.set_io_thread_count(io)


def get_dataset_fragments(dataset: pq.ParquetDataset, filters: ds.Expression | None = None) -> list[ds.Fragment]:
    inner = dataset._dataset  # noqa: SLF001 - pq.ParquetDataset wraps a pyarrow.dataset.Dataset
    return list(inner.get_fragments(filters) if filters is not None else inner.get_fragments())


def split_fragment_in_row_groups(fragment: ds.Fragment) -> list[ds.Fragment]:
    return list(fragment.split_by_row_group())


def add_fragments_trace(table: pa.Table, fragment: ds.Fragment) -> pa.Table:
    groups = fragment.row_groups
    ids = np.repeat(np.array([g.id for g in groups], dtype=np.int32), [g.num_rows for g in groups])
    if len(ids) != len(table):
        raise ValueError("The table does not have the number of rows of its fragment.")
    index = np.concatenate([np.arange(g.num_rows, dtype=np.int32) for g in groups]) if groups else np.zeros(0, np.int32)
    table = table.append_column("__row_groups_ids", pa.array(ids, type=pa.int32()))
    return table.append_column("__index_in_fragement", pa.array(index, type=pa.int32()))


def add_partitioning_values(table: pa.Table, fragment: ds.Fragment, columns: list[str] | None) -> pa.Table:
    """A fragment read on its own does not carry its hive partition columns; append them as dictionary columns."""
    for key, value in ds.get_partition_keys(fragment.partition_expression).items():
        if (columns is None or key in columns) and key not in table.column_names:
            col = pa.DictionaryArray.from_arrays(np.zeros(len(table), dtype=np.int32), pa.array([value]))
            table = table.append_column(key, col)
    return table


def rename_table_columns(table: pa.Table, mapper: dict[str, str]) -> pa.Table:
    return table.rename_columns([mapper.get(name, name) for name in table.column_names])


def _remove_quietly(path: str) -> None:
    try:
        os.remove(path)
    except FileNotFoundError:
        pass


def table_to_mmap_table(table: pa.Table, cache_dir: str) -> pa.Table:
    """Writes ``table`` to an Arrow IPC file in ``cache_dir`` and returns a memory-mapped view; the file is removed
    when the returned table is garbage collected."""
    path = str(Path(cache_dir) / f"table_{uuid.uuid4().hex[:15]}.arrow")
    with pa.OSFile(path, "wb") as sink, pa.ipc.new_stream(sink, table.schema) as writer:
        writer.write_table(table)
    with pa.memory_map(path, "rb") as source:
        mapped = pa.ipc.open_stream(source).read_all()
    weakref.finalize(mapped, _remove_quietly, path)
    return mapped


def compute_rows_length(column: pa.Array | pa.ChunkedArray) -> np.ndarray:
    """Per-row length of a list or string column (other types count 1 per row)."""
    arr = pyarrow_column_to_array(column)
    t = arr.type
    import pyarrow.compute as pc

    if pa.types.is_list(t) or pa.types.is_large_list(t):
        return np.asarray(pc.list_value_length(arr).to_numpy(zero_copy_only=False), dtype=np.int64)
    if pa.types.is_fixed_size_list(t):
        return np.full(len(arr), t.list_size, dtype=np.int64)
    if pa.types.is_string(t) or pa.types.is_large_string(t):
        return np.asarray(pc.utf8_length(arr).to_numpy(zero_copy_only=False), dtype=np.int64)
    return np.ones(len(arr), dtype=np.int64)
