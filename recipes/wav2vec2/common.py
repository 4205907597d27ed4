"""Manifest-based speech dataset shared by the wav2vec 2.0 recipes (cf. fairseq2
``recipes/wav2vec2/ssl/data/dataset.py:74-339``, ``recipes/wav2vec2/asr/data/dataset.py``,
``.../data/preprocessing.py``, ``.../data/batch_utils.py``).

``<split>.tsv``: the first line is the audio root directory, every other line is
``relative/path.wav<TAB>num_frames``. ASR splits also have ``<split>.wrd`` with one transcript per
line, aligned with the manifest. Examples are bucketed by length so that a batch holds at most
``max_num_elements`` frames, audio is optionally normalised to zero mean / unit variance, and SSL
batches are cropped to the shortest utterance (no padding enters the contrastive loss).
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Final

import torch
from torch import Tensor
from torch.nn.functional import layer_norm

from fairseq2_b200.data import Collater, DataPipeline, FileMapper, create_bucket_sizes, read_sequence
from fairseq2_b200.data.audio import AudioDecoder
from fairseq2_b200.data.tokenizers import Tokenizer
from fairseq2_b200.datasets import DataPipelineReader, DatasetError, DataReadError, Seq2SeqBatch, SequenceBatch, SyncMode
from fairseq2_b200.gang import Gangs
from fairseq2_b200.recipe.config import DatasetSection

WAV2VEC2_SSL_DATASET: Final = "wav2vec2_ssl"
WAV2VEC2_ASR_DATASET: Final = "wav2vec2_asr"


@dataclass(kw_only=True)
class ManifestDatasetConfig:
    path: Path = Path()
    """The directory holding the ``<split>.tsv`` (and ``<split>.wrd``) files."""


@dataclass(kw_only=True)
class SpeechDatasetSection(DatasetSection):
    train_split: str | None = "train"
    valid_split: str | None = "valid"
    min_audio_len: int = 32_000
    max_audio_len: int = 250_000
    max_num_elements: int = 1_500_000
    """Audio frames per batch."""
    normalize_audio: bool = False
    example_shuffle_window: int = 0
    batch_shuffle_window: int = 0
    num_prefetch: int = 4
    npc: int = 10
    no_padding: bool = True
    """SSL only: crop every utterance of a batch to the shortest one instead of padding."""


class ManifestSpeechDataset:
    def __init__(self, name: str, manifest_dir: Path) -> None:
        self._name, self._dir = name, Path(manifest_dir)
        if not self._dir.is_dir():
            raise DatasetError(f"'{self._dir}' is not a directory.")
        self._splits = {f.stem for f in self._dir.glob("*.tsv")}
        if not self._splits:
            raise DatasetError(f"No .tsv manifest found under '{self._dir}'.")

    def splits(self) -> set[str]:
        return set(self._splits)

    def _read_manifest(self, split: str, with_text: bool) -> tuple[Path, list[dict[str, Any]]]:
        if split not in self._splits:
            raise DataReadError(f"'{split}' is not a known split; available: {sorted(self._splits)}.")
        lines = (self._dir / f"{split}.tsv").read_text(encoding="utf-8").splitlines()
        if not lines:
            raise DatasetError(f"The manifest of the '{split}' split is empty.")
        root = Path(lines[0].strip())
        rows = []
        for ln in lines[1:]:
            if not ln.strip():
                continue
            f = ln.split("\t")
            rows.append({"audio": f[0], "audio_size": int(f[1])})
        if with_text:
            wrd = self._dir / f"{split}.wrd"
            if not wrd.exists():
                raise DatasetError(f"The transcript file '{wrd}' of the '{split}' split does not exist.")
            texts = wrd.read_text(encoding="utf-8").splitlines()
            if len(texts) != len(rows):
                raise DatasetError(f"'{wrd}' has {len(texts)} lines, but the manifest has {len(rows)} utterances.")
            for r, t in zip(rows, texts):
                r["text"] = t
        return root, rows

    def create_reader(self, split: str, gangs: Gangs, section: SpeechDatasetSection, *, tokenizer: Tokenizer | None = None,
                      train: bool = True, seed: int = 2, num_accumulate: int = 1, dtype: torch.dtype = torch.float32
                      ) -> DataPipelineReader[Any]:
        asr = tokenizer is not None
        root, rows = self._read_manifest(split, with_text=asr)
        b = read_sequence(rows)
        if train and section.example_shuffle_window != 1:
            b.shuffle(section.example_shuffle_window, seed=seed)
        b.shard(gangs.dp.rank, gangs.dp.size, allow_uneven=True)
        sizes = create_bucket_sizes(min_seq_len=section.min_audio_len, max_seq_len=section.max_audio_len,
                                    max_num_elements=section.max_num_elements, num_seqs_multiple_of=1)
        b.bucket_by_length(sizes, selector="audio_size", min_data_len=section.min_audio_len,
                           skip_below_min_examples=True, skip_above_max_examples=True, drop_remainder=False)
        if train and section.batch_shuffle_window != 1:
            b.shuffle(section.batch_shuffle_window, seed=seed + 1)
        mapper = FileMapper(str(root), cached_fd_count=256)
        decoder = AudioDecoder(dtype=torch.float32)
        normalize = section.normalize_audio
        encoder = tokenizer.create_encoder() if asr else None

        def load(bucket: list[dict[str, Any]]) -> list[dict[str, Any]]:
            out = []
            for ex in bucket:
                wav = decoder(mapper(ex["audio"])["data"])["waveform"]
                if wav.ndim > 1:
                    wav = wav.mean(dim=-1)
                if normalize:
                    wav = layer_norm(wav, wav.shape)
                item: dict[str, Any] = {"audio": wav.to(dtype)}
                if encoder is not None:
                    item["text"] = encoder(ex["text"])
                out.append(item)
            return out

        b.map(load, num_parallel_calls=section.npc)
        crop = (not asr) and section.no_padding

        def crop_to_shortest(bucket: list[dict[str, Any]]) -> list[dict[str, Any]]:
            n = min(int(ex["audio"].shape[0]) for ex in bucket)
            out = []
            for ex in bucket:
                extra = int(ex["audio"].shape[0]) - n
                start = int(torch.randint(0, extra + 1, ()).item()) if (extra > 0 and train) else 0
                out.append({**ex, "audio": ex["audio"][start:start + n]})
            return out

        if crop:
            b.map(crop_to_shortest)
        pad_idx = tokenizer.vocab_info.pad_idx if asr else 0
        b.map(Collater(pad_value=pad_idx if pad_idx is not None else 0))
        b.prefetch(section.num_prefetch)

        def to_batch(ex: dict[str, Any]) -> Any:
            audio = ex["audio"]
            seqs: Tensor = audio["seqs"]
            if seqs.is_floating_point() and audio.get("is_ragged", False) and not crop:
                pass
            if asr:
                text = ex["text"]
                return Seq2SeqBatch(seqs, audio["seq_lens"], text["seqs"], text["seq_lens"], example=ex)
            return SequenceBatch(seqs, audio["seq_lens"], example=ex)

        b.map(to_batch)
        return DataPipelineReader(self._name, split, b.and_return(), gangs.dp, num_accumulate=num_accumulate,
                                  drop_remainder=False, sync=True,
                                  sync_mode=SyncMode.UNTIL_FIRST if train else SyncMode.UNTIL_LAST)


def open_manifest_dataset(name: str, config: ManifestDatasetConfig) -> ManifestSpeechDataset:
    return ManifestSpeechDataset(name, config.path)
