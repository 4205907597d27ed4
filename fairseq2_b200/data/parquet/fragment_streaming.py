"""Stage 1: turn a Parquet dataset into an (optionally infinite, shuffled, rank-sharded) stream of fragments.

A *fragment* is a file or one row group of a file (``pyarrow.dataset.Fragment``): cheap to list, loaded later by
stage 2. Three shuffling regimes (``fragment_shuffle_window``):

* ``0``  -- dataset order; every rank takes fragments ``rank, rank + world, ...``.
* ``-1`` -- all fragments listed up front, a fresh global permutation per epoch (same on every rank), then
  strided sharding.
* ``n``  -- files are permuted per epoch, split into row groups on the fly and shuffled in a window of ``n``.
  With ``files_circular_shift`` each rank starts at its own position of the file list and keeps the fragments
  whose stable hash maps to it; otherwise the window output is sharded by position.

The whole stage is a ``DataPipelineBuilder``, so its position is part of the pipeline ``state_dict``
(fairseq2 ``data/parquet/fragment_streaming/primitives.py:40-622``, ``builder.py:20-129``).
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import numpy as np
import pyarrow.dataset as ds
import pyarrow.parquet as pq

from fairseq2_b200.data.data_pipeline import DataPipeline, DataPipelineBuilder, read_sequence
from fairseq2_b200.data.parquet.arrow_transform import process_filter
from fairseq2_b200.data.parquet.config import FragmentStreamingConfig, ParquetDatasetLimitOptions
from fairseq2_b200.data.parquet.utils import (
    circular_shift_left,
    fragment_stable_hash,
    get_dataset_fragments,
    split_fragment_in_row_groups,
)


def init_parquet_dataset(parquet_path: str | list[str], partition_filters: Any = None, filesystem: Any = None) -> pq.ParquetDataset:
    """Opens the dataset (metadata only). ``partition_filters`` prunes hive partitions at listing time."""
    if isinstance(filesystem, str):
        import fsspec  # noqa: F401 - names available to the expression
        import pyarrow.fs as pafs  # noqa: F401

        filesystem = eval(filesystem, {"fsspec": fsspec, "pafs": pafs})  # noqa: S307 - the documented config format
    if filesystem is None and isinstance(parquet_path, str) and "://" in parquet_path:
        from pyarrow.fs import FileSystem

        filesystem, parquet_path = FileSystem.from_uri(parquet_path)
    return pq.ParquetDataset(parquet_path, filters=process_filter(partition_filters), filesystem=filesystem)


def list_parquet_fragments(dataset: pq.ParquetDataset, limit: ParquetDatasetLimitOptions | None = None,
                           split_to_row_groups: bool = True, filters: Any = None) -> list[ds.Fragment]:
    """File fragments (sorted by path), cut down by ``limit``, optionally expanded to row groups."""
    files = sorted(get_dataset_fragments(dataset, process_filter(filters)), key=lambda f: f.path)
    if limit is not None:
        if limit.fraction_of_files is not None:
            files = files[: max(1, int(round(limit.fraction_of_files * len(files))))]
        if limit.nb_files is not None:
            files = files[: limit.nb_files]
    if not split_to_row_groups:
        fragments = files
    else:
        fragments = [g for f in files for g in split_fragment_in_row_groups(f)]
    if limit is not None:
        if limit.nb_fragments is not None:
            fragments = fragments[: limit.nb_fragments]
        if limit.nb_rows is not None:
            kept, rows = [], 0
            for frag in fragments:
                if rows >= limit.nb_rows:
                    break
                kept.append(frag)
                rows += sum(g.num_rows for g in frag.row_groups) if frag.row_groups is not None else frag.count_rows()
            fragments = kept
    return fragments


def _epochs(nb_epochs: int | None) -> DataPipelineBuilder:
    return DataPipeline.count() if nb_epochs is None else read_sequence(list(range(nb_epochs)))


def stream_parquet_fragments(dataset: pq.ParquetDataset, *, nb_epochs: int | None, seed: int = 123,
                             shuffle_window: int = 0, split_to_row_groups: bool = True,
                             limit: ParquetDatasetLimitOptions | None = None, files_circular_shift: bool = False,
                             partition_filters: Any = None, rank: int = 0, world_size: int = 1) -> DataPipelineBuilder:
    if shuffle_window < -1:
        raise ValueError(f"`shuffle_window` must be -1, 0 or positive, but is {shuffle_window} instead.")
    if not 0 <= rank < world_size:
        raise ValueError(f"`rank` must be in [0, {world_size}), but is {rank} instead.")

    if shuffle_window <= 0:
        fragments = list_parquet_fragments(dataset, limit, split_to_row_groups, partition_filters)
        if not fragments:
            raise ValueError("The dataset has no fragments after filtering.")

        def one_epoch(epoch: int) -> DataPipeline:
            order = fragments
            if shuffle_window == -1:
                perm = np.random.default_rng([seed, int(epoch)]).permutation(len(fragments))
                order = [fragments[i] for i in perm]
            return read_sequence(order).shard(rank, world_size, allow_uneven=True).and_return()

        return _epochs(nb_epochs).yield_from(one_epoch)

    # windowed regime: row-group metadata of a file is only read when the stream reaches it
    files = list_parquet_fragments(dataset, limit, split_to_row_groups=False, filters=partition_filters)
    if not files:
        raise ValueError("The dataset has no fragments after filtering.")
    expand: Callable[[ds.Fragment], DataPipeline]
    if split_to_row_groups:
        expand = lambda f: read_sequence(split_fragment_in_row_groups(f)).and_return()  # noqa: E731
    else:
        expand = lambda f: read_sequence([f]).and_return()  # noqa: E731

    def one_epoch_windowed(epoch: int) -> DataPipeline:
        perm = np.random.default_rng([seed, int(epoch)]).permutation(len(files))
        order = [files[i] for i in perm]
        if files_circular_shift:
            order = circular_shift_left(order, rank * len(order) // world_size)
        b = read_sequence(order).yield_from(expand)
        if files_circular_shift:
            if world_size > 1:
                b = b.filter(lambda frag: fragment_stable_hash(frag, seed + int(epoch)) % world_size == rank)
            return b.shuffle(shuffle_window, seed=seed + int(epoch) + 7919 * rank).and_return()
        return b.shuffle(shuffle_window, seed=seed + int(epoch)).shard(rank, world_size, allow_uneven=True).and_return()

    return _epochs(nb_epochs).yield_from(one_epoch_windowed)


class RejectionDistributionSmoother:
    """Rejection sampling over fragments that flattens a skewed distribution of partition groups.

    Use as ``pipeline.map(smoother).filter(lambda f: f is not None)`` on a dataset that is hive-partitioned on
    ``partition_groups``. The smoother keeps a running row count per group (the tuple of the fragment's values
    of those partition columns). A fragment of group g is accepted with probability ``p(g) ** alpha`` where
    ``p(g) = (1 / count_g) / sum_h (1 / max(count_h, min_count))`` -- the share g would have if every group were
    equally frequent. ``alpha = 0`` keeps the original distribution, ``alpha = 1`` makes it uniform over groups;
    ``min_count`` stops a group seen only a few times from dominating the normalisation.
    """

    def __init__(self, partition_groups: list[str], alpha: float = 0.5, min_count: int = 10, seed: int | None = 0) -> None:
        self.partition_groups = list(partition_groups)
        self.alpha, self.min_count = alpha, min_count
        self.freqs: dict[tuple[Any, ...], int] = {}
        self._rng = np.random.default_rng(seed)

    def extract(self, fragment: ds.Fragment) -> tuple[tuple[Any, ...], int]:
        keys = ds.get_partition_keys(fragment.partition_expression)
        group = tuple(keys.get(name) for name in self.partition_groups)
        return group, sum(g.num_rows for g in fragment.row_groups)

    def __call__(self, fragment: ds.Fragment) -> ds.Fragment | None:
        group, rows = self.extract(fragment)
        count = self.freqs[group] = self.freqs.get(group, 0) + rows
        norm = sum(1.0 / max(c, self.min_count) for c in self.freqs.values())
        accept = 1.0 / (max(count, 1) * norm)
        return fragment if self._rng.random() < accept ** self.alpha else None


class ParquetFragmentStreamer:
    def __init__(self, config: FragmentStreamingConfig) -> None:
        self.config = config
        self._dataset: pq.ParquetDataset | None = None

    @property
    def dataset(self) -> pq.ParquetDataset:
        if self._dataset is None:
            c = self.config
            self._dataset = init_parquet_dataset(c.parquet_path, c.partition_filters, c.filesystem)
        return self._dataset

    @property
    def full_schema(self) -> Any:
        return self.dataset.schema

    def build_pipeline(self, rank: int = 0, world_size: int = 1, even_sharding: bool = False) -> DataPipelineBuilder:
        """``even_sharding`` repeats each rank's share so all ranks see the same number of fragments per epoch in
        the non-windowed regimes (needed when ranks must iterate in lock step over a finite dataset)."""
        c = self.config
        if even_sharding and c.fragment_shuffle_window <= 0 and world_size > 1:
            fragments = list_parquet_fragments(self.dataset, c.limit, c.split_to_row_groups, c.partition_filters)
            per_rank = -(-len(fragments) // world_size)

            def one_epoch(epoch: int) -> DataPipeline:
                order = fragments
                if c.fragment_shuffle_window == -1:
                    perm = np.random.default_rng([c.seed, int(epoch)]).permutation(len(fragments))
                    order = [fragments[i] for i in perm]
                mine = [order[(rank + i * world_size) % len(order)] for i in range(per_rank)]
                return read_sequence(mine).and_return()

            return _epochs(c.nb_epochs).yield_from(one_epoch)
        return stream_parquet_fragments(self.dataset, nb_epochs=c.nb_epochs, seed=c.seed,
                                        shuffle_window=c.fragment_shuffle_window,
                                        split_to_row_groups=c.split_to_row_groups, limit=c.limit,
                                        files_circular_shift=c.files_circular_shift,
                                        partition_filters=c.partition_filters, rank=rank, world_size=world_size)
