"""Instruction-tuning dataset (cf. fairseq2 ``recipes/lm/sft/dataset.py:36-355``).

Sources are JSONL files (or directories of them) whose lines hold ``src`` and
``tgt`` texts (or ``chat`` messages in chat mode). Every example becomes token
indices plus a target mask that is true on the response. Batches are built in
one of three ways:

* ``PackedBatching`` (the B200 path): examples are packed back to back into a
  fixed-size pinned buffer of ``max_num_elements`` tokens; attention is
  block-diagonal over the packed sequences, so no FLOP is spent on padding and
  every step has the same shape.
* ``LengthBatching``: bucket by length so that a padded batch has at most
  ``max_num_elements`` elements.
* ``StaticBatching``: a fixed number of examples per batch.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Final

import torch

from fairseq2_b200.assets import AssetDownloadManager
from fairseq2_b200.data import Collater, CollateOptionsOverride, DataPipeline, create_bucket_sizes, read_sequence
from fairseq2_b200.data.text import read_text
from fairseq2_b200.data.tokenizers import Tokenizer
from fairseq2_b200.datasets import DataPipelineReader, SequenceBatch, SyncMode
from fairseq2_b200.gang import Gangs

LM_SFT_DATASET: Final = "lm_sft"


@dataclass
class StaticBatching:
    batch_size: int


@dataclass
class LengthBatching:
    max_num_elements: int


@dataclass
class PackedBatching:
    max_num_elements: int


Batching = StaticBatching | LengthBatching | PackedBatching


@dataclass(kw_only=True)
class LMSFTDataSource:
    path: str
    split: str | None = None
    weight: float = 1.0


@dataclass(kw_only=True)
class LMSFTDatasetConfig:
    sources: dict[str, list[LMSFTDataSource]] = field(default_factory=dict)


@dataclass(kw_only=True)
class DataReadOptions:
    batching: Batching = field(default_factory=lambda: StaticBatching(1))
    example_shuffle_window: int = 0
    batch_shuffle_window: int = 0
    drop_remainder: bool = False
    sync_batches: bool = True
    sync_mode: SyncMode = SyncMode.UNTIL_FIRST
    max_num_batches: int | None = None
    num_accumulate: int = 1
    prefetch: int = 1
    npc: int = 10
    seed: int = 2
    source_encode_mode: str = "prompt"
    target_encode_mode: str = "prompt_response"
    chat_mode: bool = False


class LMSFTDataset:
    def __init__(self, name: str, sources: dict[str, list[LMSFTDataSource]]) -> None:
        self._name, self._sources = name, sources

    def splits(self) -> list[str]:
        return sorted(self._sources)

    def _path_reader(self, path: str, split: str | None, gangs: Gangs, window: int, seed: int) -> DataPipeline:
        local = AssetDownloadManager().download_dataset(path, self._name) if "://" in path else Path(path)
        if split:
            local = local / split
        files = sorted(f for f in local.glob("**/*.jsonl") if f.is_file()) if local.is_dir() else [local]
        if not files:
            raise FileNotFoundError(f"No JSONL file found under '{local}'.")
        b = read_sequence([str(f) for f in files])
        b.yield_from(lambda f: read_text(f, rtrim=True, skip_empty=True).map(json.loads).and_return())
        if window != 1:
            b.shuffle(window, seed=seed)
        b.shard(gangs.dp.rank, gangs.dp.size, allow_uneven=True)
        return b.and_return()

    def create_reader(self, split: str, tokenizer: Tokenizer, gangs: Gangs, min_seq_len: int, max_seq_len: int,
                      options: DataReadOptions | None = None) -> DataPipelineReader[SequenceBatch]:
        o = options or DataReadOptions()
        try:
            sources = self._sources[split]
        except KeyError:
            raise ValueError(f"'{split}' is not a known split; available: {self.splits()}.") from None
        seed = o.seed
        pipes, weights = [], []
        for s in sources:
            pipes.append(self._path_reader(s.path, s.split, gangs, o.example_shuffle_window, seed))
            weights.append(s.weight)
            seed += 1
        seed += gangs.dp.rank
        b = DataPipeline.sample(pipes, weights, seed=seed) if len(pipes) > 1 else _rewrap(pipes[0])

        if o.chat_mode:
            enc = tokenizer.create_encoder()
            if not hasattr(enc, "apply_chat_template"):
                raise RuntimeError("A Hugging Face tokenizer with a chat template is required when `chat_mode` is set.")

            def encode_chat(ex: dict[str, Any]) -> dict[str, Any]:
                chat = ex.get("chat") or [{"role": "user", "content": ex.get("src")},
                                           {"role": "assistant", "content": ex.get("tgt")}]
                out = enc.apply_chat_template(chat, return_dict=True, return_assistant_tokens_mask=True,
                                              return_tensors="pt")
                return {"id": ex.get("id"), "indices": out["input_ids"][0],
                        "target_mask": out["assistant_masks"][0].bool()}

            b.map(encode_chat)
        else:
            src_enc = tokenizer.create_encoder(mode=o.source_encode_mode)
            tgt_enc = tokenizer.create_encoder(mode=o.target_encode_mode)

            def encode(ex: dict[str, Any]) -> dict[str, Any]:
                s, t = src_enc(ex["src"]), tgt_enc(ex["tgt"])
                idx = torch.cat([s, t])
                return {"id": ex.get("id"), "indices": idx, "target_mask": torch.arange(len(idx)) >= len(s)}

            b.map(encode, num_parallel_calls=o.npc)

        pad_idx = tokenizer.vocab_info.pad_idx
        bt = o.batching
        if isinstance(bt, PackedBatching):
            # the mask rides along in the sign: prompt positions are stored as -(index + 1)
            def fold(ex: dict[str, Any]) -> torch.Tensor:
                idx = ex["indices"].to(torch.int64)
                return torch.where(ex["target_mask"], idx, -(idx + 1))

            b.filter(lambda ex: min_seq_len <= len(ex["indices"]) <= max_seq_len)
            b.map(fold)
            pad = pad_idx if pad_idx is not None else 0
            b.pack(bt.max_num_elements, max_seq_len, pad_value=-(pad + 1), truncate=False,
                   drop_remainder=o.drop_remainder, pinned_memory=torch.cuda.is_available())
            if o.batch_shuffle_window != 1:
                b.shuffle(o.batch_shuffle_window, seed=seed)
            if o.max_num_batches is not None:
                b.take(o.max_num_batches)
            b.prefetch(o.prefetch)

            def to_packed(ex: dict[str, Any]) -> SequenceBatch:
                folded = ex["seqs"]
                mask = folded >= 0
                seqs = torch.where(mask, folded, -folded - 1)
                return SequenceBatch(seqs, list(ex["seq_lens"]), packed=True, target_mask=mask)

            b.map(to_packed)
        else:
            if pad_idx is None:
                raise RuntimeError("The tokenizer must define a pad token for padded batching.")
            if isinstance(bt, LengthBatching):
                sizes = create_bucket_sizes(min_seq_len=min_seq_len, max_seq_len=max_seq_len,
                                            max_num_elements=bt.max_num_elements)
                b.bucket_by_length(sizes, selector="indices", min_data_len=min_seq_len, skip_above_max_examples=True,
                                   drop_remainder=o.drop_remainder)
            else:
                b.filter(lambda ex: min_seq_len <= len(ex["indices"]) <= max_seq_len)
                b.bucket(bt.batch_size, drop_remainder=o.drop_remainder)
            if o.batch_shuffle_window != 1:
                b.shuffle(o.batch_shuffle_window, seed=seed)
            b.map(Collater(pad_value=pad_idx, overrides=[CollateOptionsOverride("target_mask", pad_value=False)]),
                  num_parallel_calls=o.npc)
            if o.max_num_batches is not None:
                b.take(o.max_num_batches)
            b.prefetch(o.prefetch)

            def to_batch(ex: dict[str, Any]) -> SequenceBatch:
                ind = ex["indices"]
                return SequenceBatch(ind["seqs"], ind["seq_lens"], target_mask=ex["target_mask"]["seqs"].bool(),
                                     example=ex)

            b.map(to_batch)
        return DataPipelineReader(self._name, split, b.and_return(), gangs.dp, num_accumulate=o.num_accumulate,
                                  drop_remainder=o.drop_remainder, sync=o.sync_batches, sync_mode=o.sync_mode)


def _rewrap(p: DataPipeline) -> Any:
    """A builder that continues from an already built pipeline."""
    return DataPipeline.concat([p])


def open_lm_sft_dataset(name: str, config: LMSFTDatasetConfig) -> LMSFTDataset:
    return LMSFTDataset(name, config.sources)
