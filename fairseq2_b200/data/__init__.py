"""Data pipeline API backed by the native runtime ``fairseq2_b200._data``
(C++; cf. fairseq2 ``data/data_pipeline.py`` and ``fairseq2n``)."""
from fairseq2_b200.data.data_pipeline import (ByteStreamError, CollateOptionsOverride, Collater, DataPipeline,
                                              DataPipelineBuilder, DataPipelineError, FileMapper, MemoryBlock,
                                              RecordError, SequenceData, create_bucket_sizes,
                                              get_last_failed_example, list_files, read_iterator, read_sequence,
                                              read_zipped_records)
