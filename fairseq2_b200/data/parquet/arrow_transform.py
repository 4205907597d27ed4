"""Table-level Arrow transforms (fairseq2 ``data/parquet/arrow_transform.py:20-312``)."""

from __future__ import annotations

from typing import Any

import numpy as np
import pyarrow as pa
import pyarrow.compute as pc
import pyarrow.dataset as ds

from fairseq2_b200.data.parquet.utils import compute_rows_length, pyarrow_column_to_array


def process_filter(filters: Any) -> ds.Expression | None:
    """``None`` | expression | string | list of those -> one AND-ed expression. Strings are evaluated with ``pa``,
    ``pc`` and ``ds`` in scope."""
    if filters is None:
        return None
    if isinstance(filters, str):
        return eval(filters, {"pa": pa, "pc": pc, "ds": ds})  # noqa: S307 - the documented config format
    if isinstance(filters, (list, tuple)):
        parts = [process_filter(f) for f in filters]
        parts = [p for p in parts if p is not None]
        if not parts:
            return None
        out = parts[0]
        for p in parts[1:]:
            out = out & p
        return out
    return filters


def apply_filter(table: pa.Table, filters: Any = None, drop_null: bool = True) -> pa.Table:
    if drop_null:
        table = table.drop_null()
    expr = process_filter(filters)
    if expr is not None:
        table = table.filter(expr)
    return table


def concat_table(tables: list[pa.Table], combine: bool = True) -> pa.Table:
    """Concatenates tables whose schemas agree up to column order and dictionary encoding."""
    if not tables:
        raise ValueError("`tables` must not be empty.")
    names = tables[0].column_names
    aligned = []
    for t in tables:
        t = t.select(names)
        for i, field in enumerate(t.schema):
            if pa.types.is_dictionary(field.type):
                t = t.set_column(i, field.name, pc.cast(t[field.name], field.type.value_type))
        aligned.append(t)
    out = pa.concat_tables(aligned, promote_options="permissive")
    return out.combine_chunks() if combine else out


def replace_table_column(table: pa.Table, name: str, column: pa.Array | pa.ChunkedArray) -> pa.Table:
    return table.set_column(table.column_names.index(name), name, column)


def maybe_cast(column: pa.Array | pa.ChunkedArray, target: pa.DataType) -> pa.Array | pa.ChunkedArray:
    return column if column.type == target else pc.cast(column, target)


def filter_strings_by_length(table: pa.Table, column: str, min_len: int | None = None, max_len: int | None = None) -> pa.Table:
    lengths = pc.utf8_length(table[column])
    mask: Any = None
    if min_len is not None:
        mask = pc.greater_equal(lengths, min_len)
    if max_len is not None:
        upper = pc.less_equal(lengths, max_len)
        mask = upper if mask is None else pc.and_(mask, upper)
    return table if mask is None else table.filter(mask)


def filter_list_by_range(table: pa.Table, column: str, min_val: float | None = None, max_val: float | None = None) -> pa.Table:
    """Keeps the rows whose list values ALL lie in ``[min_val, max_val]``."""
    arr = pyarrow_column_to_array(table[column])
    values = np.asarray(arr.values.to_numpy(zero_copy_only=False))
    offsets = np.asarray(arr.offsets.to_numpy())
    bad = np.zeros(len(values), dtype=np.int64)
    if min_val is not None:
        bad |= values < min_val
    if max_val is not None:
        bad |= values > max_val
    cum = np.concatenate([[0], np.cumsum(bad)])
    keep = (cum[offsets[1:]] - cum[offsets[:-1]]) == 0
    return table.filter(pa.array(keep))


def repeat_list_column(table: pa.Table, column: str, length_column: str) -> pa.Array:
    """Row i's value of ``column`` repeated ``len(table[length_column][i])`` times, as a list column."""
    lengths = compute_rows_length(table[length_column])
    values = pyarrow_column_to_array(table[column])
    taken = values.take(pa.array(np.repeat(np.arange(len(table)), lengths)))
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    return pa.ListArray.from_arrays(pa.array(offsets), taken)
