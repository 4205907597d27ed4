"""Transformer decoder stack (cf. fairseq2 ``models/transformer/decoder.py:37-230``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Iterable

import torch
from torch import Tensor
from torch.nn import Module, ModuleList

from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer.decoder_layer import TransformerDecoderLayer
from fairseq2_b200.models.transformer.encoder import _HookMixin, drop_iter
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm


class TransformerDecoder(Module, _HookMixin, ABC):
    def __init__(self) -> None:
        super().__init__()
        self._layer_hooks = {}

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, encoder_output: Tensor,
                encoder_output_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor: ...


class StandardTransformerDecoder(TransformerDecoder):
    def __init__(self, layers: Iterable[TransformerDecoderLayer], layer_norm: LayerNorm | None = None, *,
                 layer_drop_p: float = 0.0) -> None:
        super().__init__()
        self.layers = ModuleList(layers)
        self.layer_norm = layer_norm
        self.layer_drop_p = layer_drop_p
        #: source of the LayerDrop decisions (``None``: the global CPU generator, which jobs seed differently on
        #: every rank). A data-parallel engine whose collectives need every rank to run the same layers installs a
        #: generator that is seeded identically everywhere.
        self.layer_drop_generator: torch.Generator | None = None

    def forward(self, seqs, seqs_layout, encoder_output, encoder_output_layout, *, state_bag=None):  # type: ignore[override]
        self_cache, cross_cache = AttentionBiasCache(), AttentionBiasCache()
        n = len(self.layers)
        for i, layer in drop_iter(self.layers, self.layer_drop_p, self.training, self.layer_drop_generator):
            seqs = layer(seqs, seqs_layout, encoder_output, encoder_output_layout, self_cache, cross_cache,
                         state_bag=state_bag)
            stop = False
            for hook in self._layer_hooks.values():
                if not hook(i, seqs, seqs_layout, n):  # type: ignore[operator]
                    stop = True
            if stop:
                break
        if self.layer_norm is not None:
            seqs = self.layer_norm(seqs)
        return seqs
