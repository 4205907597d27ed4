"""Prompt dataset for batch generation (cf. fairseq2 ``recipes/lm/generate/dataset.py``): JSONL lines with a
``prompt`` (or ``src``) text and an optional ``id``."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Final

from fairseq2_b200.data import Collater, read_sequence
from fairseq2_b200.data.text import read_text
from fairseq2_b200.data.tokenizers import Tokenizer
from fairseq2_b200.datasets import DataPipelineReader, SequenceBatch, SyncMode
from fairseq2_b200.gang import Gangs

LM_GENERATE_DATASET: Final = "lm_generate"


@dataclass(kw_only=True)
class LMGenerateDatasetConfig:
    path: Path = Path()


class LMGenerateDataset:
    def __init__(self, name: str, path: Path) -> None:
        self._name, self._path = name, Path(path)

    def create_reader(self, tokenizer: Tokenizer, gangs: Gangs, *, batch_size: int = 1, prefetch: int = 1,
                      encode_mode: str = "prompt") -> DataPipelineReader[SequenceBatch]:
        path = self._path
        files = sorted(f for f in path.glob("**/*.jsonl") if f.is_file()) if path.is_dir() else [path]
        b = read_sequence([str(f) for f in files])
        b.yield_from(lambda f: read_text(f, rtrim=True, skip_empty=True).map(json.loads).and_return())
        b.shard(gangs.dp.rank, gangs.dp.size, allow_uneven=True)
        enc = tokenizer.create_encoder(mode=encode_mode)
        counter = iter(range(1 << 62))

        def encode(ex: dict[str, Any]) -> dict[str, Any]:
            prompt = ex.get("prompt", ex.get("src"))
            if prompt is None:
                raise ValueError("Every example must have a 'prompt' (or 'src') field.")
            id_ = ex.get("id")
            return {"id": id_ if id_ is not None else next(counter), "prompt": prompt, "indices": enc(prompt)}

        b.map(encode)
        b.bucket(batch_size)
        pad = tokenizer.vocab_info.pad_idx
        b.map(Collater(pad_value=pad if pad is not None else 0))
        b.prefetch(prefetch)

        def to_batch(ex: dict[str, Any]) -> SequenceBatch:
            ind = ex["indices"]
            return SequenceBatch(ind["seqs"], ind["seq_lens"], example=ex)

        b.map(to_batch)
        return DataPipelineReader(self._name, "default", b.and_return(), gangs.dp, drop_remainder=False, sync=True,
                                  sync_mode=SyncMode.UNTIL_LAST)


def open_lm_generate_dataset(name: str, config: LMGenerateDatasetConfig) -> LMGenerateDataset:
    return LMGenerateDataset(name, config.path)
