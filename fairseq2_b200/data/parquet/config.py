"""Configuration of the three Parquet stages: fragment streaming, fragment loading, table bucketing.

Field names follow fairseq2 ``data/parquet/fragment_streaming/config.py:16-183``,
``fragment_loading/config.py:20-160`` and ``table_bucketing/config.py:15-129`` so existing configs carry over.
"""

from __future__ import annotations

from copy import deepcopy
from dataclasses import dataclass, fields, is_dataclass
from typing import Any


@dataclass
class ParquetDatasetLimitOptions:
    """Load only a leading part of the dataset (debugging, scaling-law runs). Applied after the partition filters,
    before any shuffling; every limit that is set applies."""

    fraction_of_files: float | None = None
    nb_files: int | None = None
    nb_fragments: int | None = None
    nb_rows: int | None = None


@dataclass
class FragmentStreamingConfig:
    parquet_path: str | list[str] = ""
    """File, directory (hive-partitioned or flat) or list of files. A ``scheme://`` prefix selects the file system."""

    filesystem: Any | None = None
    """A pyarrow / fsspec file system object, or a string expression evaluating to one."""

    name: str | None = None
    weight: float = 1.0
    """Relative weight when several datasets are sampled together."""

    partition_filters: str | list[str] | Any | None = None
    """``pyarrow.dataset.Expression`` (or a string that evaluates to one with ``pa``, ``pc`` and ``ds`` in scope) over
    partition columns; several filters are AND-ed."""

    limit: ParquetDatasetLimitOptions | None = None

    split_to_row_groups: bool = True
    """Stream row groups rather than whole files."""

    seed: int = 123

    fragment_shuffle_window: int = 40
    """0: no shuffling; -1: all fragments of the dataset are shuffled globally each epoch; n > 0: files are shuffled
    each epoch and the stream of their row groups is shuffled inside a sliding window of n."""

    files_circular_shift: bool = False
    """With a positive window: rank r starts reading the (shuffled) file list at position ``r * len / world`` and
    fragments are assigned to ranks by a stable hash, so every rank walks all files but keeps a disjoint subset."""

    nb_epochs: int | None = None
    """``None`` = repeat forever."""

    def add_partition_filter(self, filters: list[Any]) -> "FragmentStreamingConfig":
        config = deepcopy(self)
        current = config.partition_filters
        if current is None:
            config.partition_filters = list(filters)
        elif isinstance(current, list):
            config.partition_filters = [*current, *filters]
        else:
            config.partition_filters = [current, *filters]
        return config


@dataclass
class NamedColumns:
    """Subclass with ``new_name: str = "column_in_file"`` fields to select and rename columns; an optional
    ``extra_columns: list[str]`` field lists columns that are loaded under their own names; ``None`` values are
    skipped."""

    def __post_init__(self) -> None:
        for f in fields(self):
            value = getattr(self, f.name)
            if f.name == "extra_columns":
                if value is not None and not (isinstance(value, list) and all(isinstance(c, str) for c in value)):
                    raise TypeError(f"Field 'extra_columns' must be a list of strings, got {type(value).__name__} instead.")
            elif value is not None and not isinstance(value, str):
                raise TypeError(f"Field '{f.name}' must be of type str, got {type(value).__name__} instead.")

    def _named(self) -> dict[str, str]:
        assert is_dataclass(self)
        return {f.name: getattr(self, f.name) for f in fields(self)
                if f.name != "extra_columns" and getattr(self, f.name) is not None}

    def get_flatten_columns(self) -> list[str]:
        cols = list(self._named().values())
        cols.extend(c for c in (getattr(self, "extra_columns", None) or []) if c is not None)
        return cols

    def get_renaming_mapper(self) -> dict[str, str]:
        return {original: new for new, original in self._named().items()}


@dataclass
class FragmentLoadingConfig:
    columns: NamedColumns | None = None
    """``None`` loads every column under its own name."""

    rename_columns: bool = True

    add_fragment_traces: bool = True
    """Append ``__row_groups_ids`` and ``__index_in_fragement`` columns so every row can be traced to its place in
    the dataset."""

    drop_null: bool = True
    min_batch_size: int = 1
    """Tables with fewer rows than this (after null dropping and filtering) are dropped."""

    filters: str | list[str] | Any | None = None
    """Row filter evaluated in memory after loading, before renaming."""

    non_deterministic_read: bool = False
    use_threads: bool = False
    nb_prefetch: int = 0
    num_parallel_fragments: int = 1

    cache: bool = False
    """Spill each loaded table to a memory-mapped Arrow file that is deleted when the table is released."""

    cache_dir: str | None = None


@dataclass
class TableBucketingConfig:
    """First concatenate loaded tables up to a target, then cut the result into batches. With all defaults the
    table stream passes through unchanged. The ``target_*`` fields are mutually exclusive."""

    min_fragment_number: int = 1
    max_fragment_number: int | None = None
    target_table_size: int | None = None
    """rows"""
    target_table_memory: int | None = None
    """MiB"""
    target_total_length: int | None = None
    """sum of the row lengths (needs ``length_columns``)"""
    combine_chunks: bool = True

    batch_size: int | None = None
    order_by_length: bool = False
    length_reducer: str = "max"
    """how the lengths of several ``length_columns`` combine per row: "max" or "sum" """
    total_batch_length: int | None = None
    """with ``order_by_length``: cap on ``rows x longest row`` of a batch (padding included)"""
    length_columns: list[str | None] | None = None
    drop_long_seq: bool = True
    shuffle: bool = False
    seed: int | None = 321

    cache: bool = False
    cache_dir: str | None = None
    nb_prefetch: int = 0
    num_parallel_calls: int = 1

    def __post_init__(self) -> None:
        targets = [t for t in (self.target_table_size, self.target_table_memory, self.target_total_length) if t is not None]
        if len(targets) > 1:
            raise ValueError("`target_table_size`, `target_table_memory` and `target_total_length` are mutually exclusive.")
        if self.length_reducer not in ("max", "sum"):
            raise ValueError(f"`length_reducer` must be 'max' or 'sum', but is '{self.length_reducer}' instead.")
        needs_len = self.order_by_length or self.target_total_length is not None or self.total_batch_length is not None
        if needs_len and not [c for c in (self.length_columns or []) if c is not None]:
            raise ValueError("`length_columns` must be given when batches are formed by length.")
