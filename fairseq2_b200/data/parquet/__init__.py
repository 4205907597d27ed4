"""Parquet datasets as data pipelines: fragment streaming -> fragment loading -> table bucketing
(fairseq2 ``data/parquet/__init__.py:46-122``)."""

from __future__ import annotations

from dataclasses import dataclass, field

from fairseq2_b200.data.data_pipeline import DataPipelineBuilder
from fairseq2_b200.data.parquet.arrow_transform import (
    apply_filter,
    concat_table,
    filter_list_by_range,
    filter_strings_by_length,
    maybe_cast,
    process_filter,
    repeat_list_column,
    replace_table_column,
)
from fairseq2_b200.data.parquet.config import (
    FragmentLoadingConfig,
    FragmentStreamingConfig,
    NamedColumns,
    ParquetDatasetLimitOptions,
    TableBucketingConfig,
)
from fairseq2_b200.data.parquet.fragment_loading import ParquetFragmentLoader, load_fragment
from fairseq2_b200.data.parquet.fragment_streaming import (
    ParquetFragmentStreamer,
    RejectionDistributionSmoother,
    init_parquet_dataset,
    list_parquet_fragments,
    stream_parquet_fragments,
)
from fairseq2_b200.data.parquet.table_bucketing import (
    TableBucketer,
    build_batching_loop_over_one_table,
    compute_length_splits,
)
from fairseq2_b200.data.parquet.utils import (
    BatchOutputType,
    NestedDict,
    NestedDictValue,
    get_dataset_fragments,
    pyarrow_column_to_array,
    pyarrow_cpu,
    pyarrow_table_to_torch_dict,
    pyarrow_to_torch_tensor,
    split_fragment_in_row_groups,
)


@dataclass
class BasicDataLoadingConfig:
    fragment_stream_config: FragmentStreamingConfig
    fragment_load_config: FragmentLoadingConfig = field(default_factory=FragmentLoadingConfig)
    """default: all columns"""
    table_bucketing_config: TableBucketingConfig = field(default_factory=TableBucketingConfig)
    """default: tables pass through as loaded"""


def build_basic_parquet_data_pipeline(config: BasicDataLoadingConfig, rank: int = 0, world_size: int = 1) -> DataPipelineBuilder:
    """Fragments -> tables -> batches (``pyarrow.Table``); convert with ``.map(pyarrow_table_to_torch_dict)``."""
    b = ParquetFragmentStreamer(config.fragment_stream_config).build_pipeline(rank=rank, world_size=world_size)
    b = ParquetFragmentLoader(config.fragment_load_config).apply(b)
    return TableBucketer(config.table_bucketing_config).apply(b)


__all__ = [
    "BasicDataLoadingConfig", "BatchOutputType", "FragmentLoadingConfig", "FragmentStreamingConfig", "NamedColumns",
    "NestedDict", "NestedDictValue", "ParquetDatasetLimitOptions", "ParquetFragmentLoader", "ParquetFragmentStreamer",
    "RejectionDistributionSmoother", "TableBucketer", "TableBucketingConfig", "apply_filter",
    "build_basic_parquet_data_pipeline", "build_batching_loop_over_one_table", "compute_length_splits", "concat_table",
    "filter_list_by_range", "filter_strings_by_length", "get_dataset_fragments", "init_parquet_dataset",
    "list_parquet_fragments", "load_fragment", "maybe_cast", "process_filter", "pyarrow_column_to_array", "pyarrow_cpu",
    "pyarrow_table_to_torch_dict", "pyarrow_to_torch_tensor", "repeat_list_column", "replace_table_column",
    "split_fragment_in_row_groups", "stream_parquet_fragments",
]
