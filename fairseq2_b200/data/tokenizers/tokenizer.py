"""Tokenizer interfaces (cf. fairseq2 ``data/tokenizers/tokenizer.py:18-114``,
``vocab_info.py:13-39``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Sequence

import torch
from torch import Tensor

from fairseq2_b200.typing import Device


@dataclass
class VocabularyInfo:
    size: int
    unk_idx: int | None = None
    bos_idx: int | None = None
    eos_idx: int | None = None
    pad_idx: int | None = None
    boh_idx: int | None = None
    eoh_idx: int | None = None

    def __post_init__(self) -> None:
        # a pad index that coincides with EOS cannot be told apart from real EOS tokens
        if self.pad_idx is not None and self.pad_idx == self.eos_idx:
            self.pad_idx = None


class TokenEncoder(ABC):
    @abstractmethod
    def __call__(self, text: str) -> Tensor: ...

    @abstractmethod
    def encode_as_tokens(self, text: str) -> list[str]: ...

    @property
    def prefix_indices(self) -> Tensor | None:
        return None

    @property
    def suffix_indices(self) -> Tensor | None:
        return None


class TokenDecoder(ABC):
    @abstractmethod
    def __call__(self, token_indices: Tensor) -> str: ...

    @abstractmethod
    def decode_from_tokens(self, tokens: Sequence[str]) -> str: ...


class Tokenizer(ABC):
    @abstractmethod
    def create_encoder(self, *, task: str | None = None, lang: str | None = None, mode: str | None = None,
                       device: Device | None = None, pin_memory: bool = False) -> TokenEncoder: ...

    @abstractmethod
    def create_raw_encoder(self, *, device: Device | None = None, pin_memory: bool = False) -> TokenEncoder: ...

    @abstractmethod
    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder: ...

    @property
    @abstractmethod
    def vocab_info(self) -> VocabularyInfo: ...


def _to_tensor(ids: Sequence[int], device: Device | None, pin_memory: bool) -> Tensor:
    t = torch.tensor(list(ids), dtype=torch.int64)
    if pin_memory and torch.cuda.is_available():
        t = t.pin_memory()
    return t.to(device, non_blocking=True) if device is not None else t
