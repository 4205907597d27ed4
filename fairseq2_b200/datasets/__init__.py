from fairseq2_b200.datasets.batch import Seq2SeqBatch, SequenceBatch
from fairseq2_b200.datasets.data_reader import DataPipelineReader, DataReader, DataReadError, SyncMode
from fairseq2_b200.datasets.family import (DatasetError, DatasetFamily, DatasetHub, UnknownDatasetError,
                                           UnknownDatasetFamilyError, get_dataset_family, open_dataset,
                                           register_dataset_family)
