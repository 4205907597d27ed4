"""Stage 2: read each fragment into a ``pyarrow.Table`` -- column selection and renaming, partition values,
trace columns, null dropping, row filters, optional mmap spill, parallel reads and prefetch
(fairseq2 ``data/parquet/fragment_loading/builder.py:30-211``)."""

from __future__ import annotations

import tempfile
from typing import Any

import pyarrow as pa
import pyarrow.dataset as ds

from fairseq2_b200.data.data_pipeline import DataPipelineBuilder
from fairseq2_b200.data.parquet.arrow_transform import apply_filter, process_filter
from fairseq2_b200.data.parquet.config import FragmentLoadingConfig
from fairseq2_b200.data.parquet.utils import (
    add_fragments_trace,
    add_partitioning_values,
    rename_table_columns,
    table_to_mmap_table,
)


def load_fragment(fragment: ds.Fragment, columns: list[str] | None = None, add_fragment_traces: bool = True,
                  use_threads: bool = False, add_partitioning_columns: bool = True) -> pa.Table:
    """One fragment -> table. Partition columns are not stored in the file: they are left out of the read and
    appended from the fragment's partition expression."""
    physical = set(fragment.physical_schema.names)
    read_cols = None if columns is None else [c for c in columns if c in physical]
    if columns is not None:
        partition_keys = set(ds.get_partition_keys(fragment.partition_expression))
        missing = [c for c in columns if c not in physical and c not in partition_keys]
        if missing:
            raise KeyError(f"The columns {missing} are not in the dataset (file '{fragment.path}').")
    table = fragment.to_table(columns=read_cols, use_threads=use_threads)
    if add_partitioning_columns:
        table = add_partitioning_values(table, fragment, columns)
    if add_fragment_traces:
        table = add_fragments_trace(table, fragment)
    return table


class ParquetFragmentLoader:
    def __init__(self, config: FragmentLoadingConfig) -> None:
        self.config = config
        self._filters = process_filter(config.filters)
        self._columns = config.columns.get_flatten_columns() if config.columns is not None else None
        self._renaming = config.columns.get_renaming_mapper() if (config.columns is not None and config.rename_columns) else None
        self._cache_dir: Any = None
        if config.cache:
            if config.cache_dir is None:
                self._tmp = tempfile.TemporaryDirectory(prefix="fs2_parquet_cache_")
                self._cache_dir = self._tmp.name
            else:
                self._cache_dir = config.cache_dir

    def load(self, fragment: ds.Fragment) -> pa.Table | None:
        c = self.config
        table = load_fragment(fragment, self._columns, c.add_fragment_traces, c.use_threads)
        table = apply_filter(table, self._filters, c.drop_null)
        if len(table) < c.min_batch_size:
            return None
        if self._renaming:
            table = rename_table_columns(table, self._renaming)
        if self._cache_dir is not None:
            table = table_to_mmap_table(table, self._cache_dir)
        return table

    def apply(self, fragment_pipeline: DataPipelineBuilder) -> DataPipelineBuilder:
        c = self.config
        b = fragment_pipeline.map(self.load, num_parallel_calls=max(c.num_parallel_fragments, 1),
                                  deterministic=not c.non_deterministic_read)
        b = b.filter(lambda t: t is not None)
        if c.nb_prefetch > 0:
            b = b.prefetch(c.nb_prefetch)
        return b

    build_pipeline = apply
