"""Sequence feature extractor interface (cf. fairseq2 ``models/feature_extractor.py:17-40``)."""
from __future__ import annotations

from abc import ABC, abstractmethod

from torch import Tensor
from torch.nn import Module

from fairseq2_b200.nn.batch_layout import BatchLayout


class SequenceFeatureExtractor(Module, ABC):
    """Turns ``(N, S, *)`` raw sequences into ``(N, S_out, feature_dim)`` features."""

    def __init__(self, feature_dim: int) -> None:
        super().__init__()
        self.feature_dim = feature_dim

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout]: ...
