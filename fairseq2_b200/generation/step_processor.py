"""Step processors that edit next-token probabilities in place
(cf. fairseq2 ``generation/step_processor.py:37-176``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Sequence

import torch
from torch import Tensor

from fairseq2_b200.ops.sampling import ngram_repeat_block


class StepProcessor(ABC):
    @abstractmethod
    def __call__(self, seqs: Tensor, probs: Tensor, lprob: bool = False) -> None:
        """``seqs``: ``(N, S)`` generated so far; ``probs``: ``(N, V)`` next-step
        (log-)probabilities, modified in place."""


class BannedSequenceProcessor(StepProcessor):
    """Prevents the listed token sequences from being generated."""

    def __init__(self, banned_seqs: Sequence[Tensor]) -> None:
        self._single: Tensor | None = None
        self._multi: list[Tensor] = []
        singles = [int(b[0]) for b in banned_seqs if b.numel() == 1]
        if singles:
            self._single = torch.tensor(singles, dtype=torch.int64)
        self._multi = [b.to(torch.int64) for b in banned_seqs if b.numel() > 1]

    def __call__(self, seqs: Tensor, probs: Tensor, lprob: bool = False) -> None:
        ban = float("-inf") if lprob else 0.0
        if self._single is not None:
            probs[:, self._single.to(probs.device)] = ban
        for b in self._multi:
            n = b.numel() - 1
            if seqs.shape[1] < n:
                continue
            prefix = b[:-1].to(seqs.device)
            hit = (seqs[:, -n:] == prefix).all(dim=1)
            probs[hit, int(b[-1])] = ban


class NGramRepeatBlockProcessor(StepProcessor):
    """Blocks tokens that would complete an n-gram already present in the sequence."""

    def __init__(self, ngram_size: int) -> None:
        if ngram_size <= 0:
            raise ValueError(f"`ngram_size` must be greater than 0, but is {ngram_size} instead.")
        self.ngram_size = ngram_size

    def __call__(self, seqs: Tensor, probs: Tensor, lprob: bool = False) -> None:
        ngram_repeat_block(seqs, probs, self.ngram_size, float("-inf") if lprob else 0.0)
