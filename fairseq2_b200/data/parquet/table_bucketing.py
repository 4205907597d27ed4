"""Stage 3: regroup the stream of loaded tables into batches.

First several tables are concatenated until a target (rows, MiB, or summed sequence length) is met; then the big
table is cut into batches: fixed ``batch_size`` slices (zero-copy), or -- with ``order_by_length`` -- rows are sorted
by length and greedily grouped so that ``rows x longest row <= total_batch_length``, which keeps padding low.
Batches of one big table can be shuffled before being emitted
(fairseq2 ``data/parquet/table_bucketing/primitives.py:20-189``, ``builder.py:20-145``).
"""

from __future__ import annotations

import tempfile
from typing import Any

import numpy as np
import pyarrow as pa

from fairseq2_b200.data.data_pipeline import DataPipeline, DataPipelineBuilder, read_sequence
from fairseq2_b200.data.parquet.arrow_transform import concat_table
from fairseq2_b200.data.parquet.config import TableBucketingConfig
from fairseq2_b200.data.parquet.utils import compute_rows_length, table_to_mmap_table


def compute_length_splits(lengths: np.ndarray, max_tokens: int, *, order_by_length: bool = True,
                          drop_long_seq: bool = True) -> list[np.ndarray]:
    """Index groups such that ``len(group) * max(lengths[group]) <= max_tokens``.

    Rows longer than ``max_tokens`` are dropped (``drop_long_seq``) or emitted alone. With ``order_by_length`` rows
    are visited from short to long (stable), otherwise in their given order.
    """
    n = len(lengths)
    order = np.argsort(lengths, kind="stable") if order_by_length else np.arange(n)
    groups: list[np.ndarray] = []
    start, longest = 0, 0
    for pos in range(n):
        length = int(lengths[order[pos]])
        if length > max_tokens:
            if start < pos:
                groups.append(order[start:pos])
            if not drop_long_seq:
                groups.append(order[pos: pos + 1])
            start, longest = pos + 1, 0
            continue
        new_longest = max(longest, length)
        if new_longest * (pos - start + 1) > max_tokens:
            groups.append(order[start:pos])
            start, longest = pos, length
        else:
            longest = new_longest
    if start < n:
        groups.append(order[start:n])
    return [g for g in groups if len(g)]


def row_lengths(table: pa.Table, columns: list[str | None], reducer: str = "max") -> np.ndarray:
    cols = [c for c in columns if c is not None]
    if not cols:
        raise ValueError("`columns` must name at least one column.")
    stacked = np.stack([compute_rows_length(table[c]) for c in cols])
    return stacked.max(axis=0) if reducer == "max" else stacked.sum(axis=0)


def build_batching_loop_over_one_table(table: pa.Table, *, order_by_length: bool = False,
                                       length_columns: list[str | None] | None = None, length_reducer: str = "max",
                                       batch_size: int | None = None, max_tokens: int | None = None,
                                       drop_long_seq: bool = True, shuffle: bool = False, seed: int | None = None,
                                       num_parallel_calls: int = 1) -> DataPipeline:
    """The batches of one (concatenated) table as a pipeline of tables."""
    if max_tokens is not None:
        lengths = row_lengths(table, length_columns or [], length_reducer)
        groups = compute_length_splits(lengths, max_tokens, order_by_length=order_by_length, drop_long_seq=drop_long_seq)
        if batch_size is not None:
            groups = [g[i: i + batch_size] for g in groups for i in range(0, len(g), batch_size)]
    else:
        n = len(table)
        if order_by_length:
            order = np.argsort(row_lengths(table, length_columns or [], length_reducer), kind="stable")
        else:
            order = None
        step = batch_size or max(n, 1)
        bounds = [(i, min(i + step, n)) for i in range(0, n, step)]
        if order is None and not shuffle:
            return read_sequence([table.slice(lo, hi - lo) for lo, hi in bounds]).and_return()
        base = order if order is not None else np.arange(n)
        groups = [base[lo:hi] for lo, hi in bounds]
    if shuffle:
        perm = np.random.default_rng(seed).permutation(len(groups))
        groups = [groups[i] for i in perm]
    take = lambda idx: table.take(pa.array(idx))  # noqa: E731
    return read_sequence(groups).map(take, num_parallel_calls=max(num_parallel_calls, 1)).and_return()


class TableBucketer:
    def __init__(self, config: TableBucketingConfig) -> None:
        self.config = config
        self._cache_dir: Any = None
        if config.cache:
            if config.cache_dir is None:
                self._tmp = tempfile.TemporaryDirectory(prefix="fs2_parquet_bucket_")
                self._cache_dir = self._tmp.name
            else:
                self._cache_dir = config.cache_dir
        self._calls = 0

    def _concat(self, tables: list[pa.Table]) -> pa.Table:
        out = concat_table(tables, combine=self.config.combine_chunks)
        if self._cache_dir is not None:
            out = table_to_mmap_table(out, self._cache_dir)
        return out

    def _split(self, table: pa.Table) -> DataPipeline:
        c = self.config
        self._calls += 1
        return build_batching_loop_over_one_table(
            table, order_by_length=c.order_by_length, length_columns=c.length_columns, length_reducer=c.length_reducer,
            batch_size=c.batch_size, max_tokens=c.total_batch_length, drop_long_seq=c.drop_long_seq, shuffle=c.shuffle,
            seed=None if c.seed is None else c.seed + self._calls, num_parallel_calls=c.num_parallel_calls)

    def apply(self, pipeline: DataPipelineBuilder) -> DataPipelineBuilder:
        c = self.config
        if c.target_table_size is not None:
            threshold, cost = float(c.target_table_size), (lambda t: float(len(t)))
        elif c.target_table_memory is not None:
            threshold, cost = float(c.target_table_memory), (lambda t: t.nbytes / 2 ** 20)
        elif c.target_total_length is not None:
            cols, red = c.length_columns or [], c.length_reducer
            threshold, cost = float(c.target_total_length), (lambda t: float(row_lengths(t, cols, red).sum()))
        else:
            threshold = None
        b = pipeline
        if threshold is not None:
            b = b.dynamic_bucket(threshold, cost, min_num_examples=c.min_fragment_number,
                                 max_num_examples=c.max_fragment_number).map(self._concat)
        elif c.min_fragment_number > 1:
            b = b.bucket(c.min_fragment_number).map(self._concat)
        needs_split = c.batch_size is not None or c.order_by_length or c.total_batch_length is not None or c.shuffle
        if needs_split:
            b = b.yield_from(self._split)
        if c.nb_prefetch > 0:
            b = b.prefetch(c.nb_prefetch)
        return b

    build_pipeline = apply
