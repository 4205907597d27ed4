"""Parquet pipelines: fragment streaming (shuffle regimes, sharding, epochs, limits), loading (columns, renaming,
traces, filters, partition values) and bucketing (concat targets, length-ordered batches)."""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import pytest
import torch

pa = pytest.importorskip("pyarrow")
import pyarrow.parquet as pq  # noqa: E402

from fairseq2_b200.data.parquet import (  # noqa: E402
    BasicDataLoadingConfig,
    FragmentLoadingConfig,
    FragmentStreamingConfig,
    NamedColumns,
    ParquetDatasetLimitOptions,
    ParquetFragmentLoader,
    ParquetFragmentStreamer,
    RejectionDistributionSmoother,
    TableBucketingConfig,
    build_basic_parquet_data_pipeline,
    compute_length_splits,
    filter_list_by_range,
    filter_strings_by_length,
    pyarrow_table_to_torch_dict,
    repeat_list_column,
)


@pytest.fixture(scope="module")
def dataset_dir(tmp_path_factory: pytest.TempPathFactory) -> Path:
    root = tmp_path_factory.mktemp("pq")
    rng = np.random.default_rng(0)
    uid = 0
    for split in ("train", "dev"):
        for lang in ("en", "fr", "de"):
            d = root / f"split={split}" / f"lang={lang}"
            d.mkdir(parents=True)
            for part in range(2):
                n = 30 if lang == "en" else 10
                lens = rng.integers(1, 12, n)
                table = pa.table({
                    "id": pa.array(np.arange(uid, uid + n), type=pa.int64()),
                    "tokens": pa.array([list(map(int, rng.integers(0, 100, k))) for k in lens], type=pa.list_(pa.int32())),
                    "text": pa.array(["w" * int(k) for k in lens]),
                    "score": pa.array([None if i % 7 == 3 else float(i) for i in range(n)], type=pa.float32()),
                })
                uid += n
                pq.write_table(table, d / f"part{part}.parquet", row_group_size=5)
    return root


def _ids(tables) -> list[int]:
    return [int(i) for t in tables for i in t["id"].to_pylist()]


def test_streaming_regimes_and_sharding(dataset_dir: Path) -> None:
    base = FragmentStreamingConfig(parquet_path=str(dataset_dir), partition_filters='pc.field("split") == "train"',
                                   nb_epochs=1, fragment_shuffle_window=0)
    frags = list(ParquetFragmentStreamer(base).build_pipeline().and_return())
    assert len(frags) == 2 * (6 + 2 + 2)                         # row groups of 5 rows
    per_rank = [list(ParquetFragmentStreamer(base).build_pipeline(r, 3).and_return()) for r in range(3)]
    keys = [{(f.path, f.row_groups[0].id) for f in fr} for fr in per_rank]
    assert sum(len(k) for k in keys) == len(frags) and len(set().union(*keys)) == len(frags)

    for window, shift in ((-1, False), (4, False), (4, True)):
        cfg = FragmentStreamingConfig(parquet_path=str(dataset_dir), partition_filters=['pc.field("split") == "train"'],
                                      nb_epochs=2, fragment_shuffle_window=window, files_circular_shift=shift, seed=5)
        got = [list(ParquetFragmentStreamer(cfg).build_pipeline(r, 2).and_return()) for r in range(2)]
        all_keys = [(f.path, f.row_groups[0].id) for fr in got for f in fr]
        assert len(all_keys) == 2 * len(frags) and len(set(all_keys)) == len(frags)   # two epochs, disjoint ranks
        again = list(ParquetFragmentStreamer(cfg).build_pipeline(0, 2).and_return())
        assert [(f.path, f.row_groups[0].id) for f in again] == [(f.path, f.row_groups[0].id) for f in got[0]]
        order = [(f.path, f.row_groups[0].id) for f in got[0]]
        assert order[: len(order) // 2] != order[len(order) // 2:] or shift      # epochs are permuted differently

    lim = FragmentStreamingConfig(parquet_path=str(dataset_dir), nb_epochs=1, fragment_shuffle_window=0,
                                  limit=ParquetDatasetLimitOptions(nb_files=3, nb_fragments=4))
    assert len(list(ParquetFragmentStreamer(lim).build_pipeline().and_return())) == 4
    whole = FragmentStreamingConfig(parquet_path=str(dataset_dir), nb_epochs=1, fragment_shuffle_window=0,
                                    split_to_row_groups=False)
    assert len(list(ParquetFragmentStreamer(whole).build_pipeline().and_return())) == 12


def test_streaming_state_dict_resumes(dataset_dir: Path) -> None:
    cfg = FragmentStreamingConfig(parquet_path=str(dataset_dir), nb_epochs=None, fragment_shuffle_window=6, seed=1)
    pipe = ParquetFragmentStreamer(cfg).build_pipeline().and_return()
    it = iter(pipe)
    for _ in range(17):
        next(it)
    state = pipe.state_dict()
    want = [(f.path, f.row_groups[0].id) for f in (next(it) for _ in range(9))]
    pipe2 = ParquetFragmentStreamer(cfg).build_pipeline().and_return()
    pipe2.load_state_dict(state)
    it2 = iter(pipe2)
    assert [(f.path, f.row_groups[0].id) for f in (next(it2) for _ in range(9))] == want


def test_loading_columns_filters_traces(dataset_dir: Path) -> None:
    @dataclass
    class Cols(NamedColumns):
        seq: str = "tokens"
        language: str = "lang"
        missing: str | None = None
        extra_columns: list[str] = field(default_factory=lambda: ["id"])

    stream = FragmentStreamingConfig(parquet_path=str(dataset_dir), nb_epochs=1, fragment_shuffle_window=0,
                                     partition_filters='(pc.field("split") == "dev") & (pc.field("lang") == "fr")')
    load = FragmentLoadingConfig(columns=Cols(), filters="pc.list_value_length(pc.field('tokens')) > 3",
                                 num_parallel_fragments=2, nb_prefetch=1)
    b = ParquetFragmentLoader(load).apply(ParquetFragmentStreamer(stream).build_pipeline())
    tables = list(b.and_return())
    assert tables and all(set(t.column_names) == {"seq", "language", "id", "__row_groups_ids", "__index_in_fragement"}
                          for t in tables)
    assert all(v == "fr" for t in tables for v in t["language"].to_pylist())
    assert all(len(s) > 3 for t in tables for s in t["seq"].to_pylist())
    with pytest.raises(TypeError):
        @dataclass
        class Bad(NamedColumns):
            x: int = 3  # type: ignore[assignment]
        Bad()

    # drop_null removes the rows whose score is null; without it they survive
    stream_all = FragmentStreamingConfig(parquet_path=str(dataset_dir), nb_epochs=1, fragment_shuffle_window=0)
    n_drop = sum(len(t) for t in ParquetFragmentLoader(FragmentLoadingConfig()).apply(
        ParquetFragmentStreamer(stream_all).build_pipeline()).and_return())
    n_keep = sum(len(t) for t in ParquetFragmentLoader(FragmentLoadingConfig(drop_null=False, cache=True)).apply(
        ParquetFragmentStreamer(stream_all).build_pipeline()).and_return())
    assert n_keep == 200 and n_drop < n_keep


def test_bucketing_and_torch_conversion(dataset_dir: Path) -> None:
    stream = FragmentStreamingConfig(parquet_path=str(dataset_dir), nb_epochs=1, fragment_shuffle_window=-1,
                                     partition_filters='pc.field("split") == "train"')
    load = FragmentLoadingConfig(drop_null=False, add_fragment_traces=False)
    plain = BasicDataLoadingConfig(stream, load)
    n_rows = sum(len(t) for t in build_basic_parquet_data_pipeline(plain).and_return())
    assert n_rows == 100

    fixed = BasicDataLoadingConfig(stream, load, TableBucketingConfig(target_table_size=40, batch_size=16))
    sizes = [len(t) for t in build_basic_parquet_data_pipeline(fixed).and_return()]
    assert sum(sizes) == 100 and max(sizes) == 16

    by_len = BasicDataLoadingConfig(stream, load, TableBucketingConfig(
        target_total_length=200, order_by_length=True, total_batch_length=48, length_columns=["tokens"], shuffle=True))
    batches = list(build_basic_parquet_data_pipeline(by_len).and_return())
    assert sorted(_ids(batches)) == sorted(_ids(build_basic_parquet_data_pipeline(plain).and_return()))
    for t in batches:
        lens = [len(x) for x in t["tokens"].to_pylist()]
        assert len(lens) * max(lens) <= 48
    d = pyarrow_table_to_torch_dict(batches[0].combine_chunks())
    assert isinstance(d["id"], torch.Tensor) and d["id"].dtype == torch.int64
    assert isinstance(d["tokens"], list) and d["tokens"][0].dtype == torch.int32
    assert isinstance(d["text"], list) and isinstance(d["text"][0], str)
    assert d["lang"] == ["en" if v == "en" else v for v in batches[0]["lang"].to_pylist()]

    with pytest.raises(ValueError):
        TableBucketingConfig(order_by_length=True)
    with pytest.raises(ValueError):
        TableBucketingConfig(target_table_size=1, target_table_memory=1)


def test_length_splits_and_transforms() -> None:
    lengths = np.array([5, 1, 9, 3, 3, 20, 2])
    groups = compute_length_splits(lengths, 10)
    flat = sorted(int(i) for g in groups for i in g)
    assert flat == [0, 1, 2, 3, 4, 6]                                  # the row of length 20 is dropped
    assert all(len(g) * lengths[g].max() <= 10 for g in groups)
    kept = compute_length_splits(lengths, 10, drop_long_seq=False)
    assert sorted(int(i) for g in kept for i in g) == list(range(7))

    t = pa.table({"v": pa.array([[1, 2], [5, 50], [], [3]], type=pa.list_(pa.int64())), "s": ["a", "bbb", "cc", "dddd"],
                  "k": [10, 20, 30, 40]})
    assert filter_list_by_range(t, "v", 0, 10)["k"].to_pylist() == [10, 30, 40]
    assert filter_strings_by_length(t, "s", 2, 3)["k"].to_pylist() == [20, 30]
    assert repeat_list_column(t, "k", "v").to_pylist() == [[10, 10], [20, 20], [], [40]]


def test_rejection_smoother_flattens(dataset_dir: Path) -> None:
    cfg = FragmentStreamingConfig(parquet_path=str(dataset_dir), partition_filters='pc.field("split") == "train"',
                                  nb_epochs=40, fragment_shuffle_window=-1)
    smoother = RejectionDistributionSmoother(["lang"], alpha=1.0, min_count=1, seed=0)
    kept = list(ParquetFragmentStreamer(cfg).build_pipeline().map(smoother).filter(lambda f: f is not None).and_return())
    rows: dict[str, int] = {}
    for f in kept:
        lang = smoother.extract(f)[0][0]
        rows[lang] = rows.get(lang, 0) + sum(g.num_rows for g in f.row_groups)
    assert set(rows) == {"en", "fr", "de"}
    assert max(rows.values()) / min(rows.values()) < 1.6                # 3:1:1 before smoothing
