"""Pre-training dataset (cf. fairseq2 ``recipes/lm/train/dataset.py:36-175``): JSONL shards with a ``text``
field, sharded by FILE over the data-parallel ranks, tokenised and packed back to back into pinned buffers of
``max_num_tokens + 1`` tokens (the extra token supplies the last next-token target)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Final

import torch
from torch import Tensor

from fairseq2_b200.data import DataPipeline, read_sequence
from fairseq2_b200.data.text import read_text
from fairseq2_b200.data.tokenizers import Tokenizer
from fairseq2_b200.datasets import DataPipelineReader, SequenceBatch, SyncMode
from fairseq2_b200.gang import Gangs

LM_TRAIN_DATASET: Final = "lm_train"


@dataclass(kw_only=True)
class LMTrainDataSource:
    path: Path
    weight: float = 1.0


@dataclass(kw_only=True)
class LMTrainDatasetConfig:
    sources: list[LMTrainDataSource] = field(default_factory=list)


class LMTrainDataset:
    def __init__(self, name: str, sources: list[LMTrainDataSource]) -> None:
        self._name, self._sources = name, sources

    def _path_reader(self, path: Path, gangs: Gangs) -> DataPipeline:
        path = Path(path)
        if path.is_dir():
            files = sorted(f for f in path.glob("**/*.jsonl") if f.is_file())
        else:
            files = [path]
        if len(files) < gangs.dp.size:
            raise ValueError(f"'{path}' holds {len(files)} file(s), fewer than the data-parallel size ({gangs.dp.size}); "
                             "split the corpus into at least one shard per rank.")
        b = read_sequence([str(f) for f in files])
        if gangs.dp.size > 1:
            b.shard(gangs.dp.rank, gangs.dp.size, allow_uneven=True)
        b.yield_from(lambda f: read_text(f, rtrim=True, skip_empty=True).map(json.loads).and_return())
        return b.and_return()

    def create_reader(self, tokenizer: Tokenizer, gangs: Gangs, *, max_seq_len: int, max_num_tokens: int,
                      num_accumulate: int = 1, seed: int = 2, prefetch: int = 1, sync_ranks: bool = True,
                      split: str = "train") -> DataPipelineReader[SequenceBatch]:
        pipes = [self._path_reader(s.path, gangs) for s in self._sources]
        weights = [s.weight for s in self._sources]
        b = DataPipeline.sample(pipes, weights, seed=seed) if len(pipes) > 1 else DataPipeline.concat(pipes)
        enc = tokenizer.create_encoder(mode="default")

        def encode(ex: dict[str, Any]) -> Tensor:
            return enc(ex["text"]).to(torch.int64)

        b.map(encode)
        b.pack(max_num_tokens + 1, max_seq_len, truncate=True, drop_remainder=True,
               pinned_memory=torch.cuda.is_available())
        b.prefetch(prefetch)
        b.map(lambda ex: SequenceBatch(ex["seqs"], list(ex["seq_lens"]), packed=True))
        return DataPipelineReader(self._name, split, b.and_return(), gangs.dp, num_accumulate=num_accumulate,
                                  sync=sync_ranks, sync_mode=SyncMode.UNTIL_FIRST)


def open_lm_train_dataset(name: str, config: LMTrainDatasetConfig) -> LMTrainDataset:
    return LMTrainDataset(name, config.sources)
