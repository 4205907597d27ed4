"""Embedding frontends (cf. fairseq2 ``models/transformer/frontend.py:104-122``)."""
from __future__ import annotations

import math
from abc import ABC, abstractmethod

from torch import Tensor
from torch.nn import Dropout, Module

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.embedding import Embedding
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder


class TransformerFrontend(Module, ABC):
    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None
                ) -> tuple[Tensor, BatchLayout]: ...


class TransformerEmbeddingFrontend(TransformerFrontend):
    def __init__(self, model_dim: int, embed: Embedding, pos_encoder: PositionEncoder | None = None, *,
                 no_scale: bool = False, layer_norm: LayerNorm | None = None, dropout_p: float = 0.0) -> None:
        super().__init__()
        self.model_dim = model_dim
        self.embed = embed
        self.scale = 1.0 if no_scale else math.sqrt(model_dim)
        self.pos_encoder = pos_encoder
        self.layer_norm = layer_norm
        self.dropout = Dropout(dropout_p) if dropout_p > 0.0 else None

    def forward(self, seqs, seqs_layout, *, state_bag=None):  # type: ignore[override]
        x = self.embed(seqs)
        if self.scale != 1.0:
            x = x * self.scale
        if self.pos_encoder is not None:
            x = self.pos_encoder(x, seqs_layout, state_bag=state_bag)
        if self.layer_norm is not None:
            x = self.layer_norm(x)
        if self.dropout is not None:
            x = self.dropout(x)
        return x, seqs_layout
