"""Transformer encoder stack (cf. fairseq2 ``models/transformer/encoder.py:34-201``): layers with
optional LayerDrop, a final layer norm, and per-layer output hooks."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Iterable, Protocol

import torch
from torch import Tensor
from torch.nn import Module, ModuleList

from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer.encoder_layer import TransformerEncoderLayer
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.normalization import LayerNorm


class TransformerEncoderLayerHook(Protocol):
    def __call__(self, layer_idx: int, layer_output: Tensor, layer_output_layout: BatchLayout,
                 num_layers: int) -> bool:
        """Return ``False`` to stop after this layer."""


class _HookMixin:
    _layer_hooks: dict[int, object]

    def register_layer_hook(self, hook):  # type: ignore[no-untyped-def]
        key = max(self._layer_hooks, default=-1) + 1
        self._layer_hooks[key] = hook
        hooks = self._layer_hooks

        class _Handle:
            def remove(self) -> None:
                hooks.pop(key, None)

        return _Handle()


class TransformerEncoder(Module, _HookMixin, ABC):
    def __init__(self) -> None:
        super().__init__()
        self._layer_hooks = {}

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> Tensor: ...


def drop_iter(layers: ModuleList, drop_p: float, training: bool, generator: torch.Generator | None = None):  # type: ignore[no-untyped-def]
    """Yields ``(index, layer)`` skipping each layer with probability ``drop_p`` while training (LayerDrop)."""
    if drop_p > 0.0 and training:
        probs = torch.rand(len(layers), generator=generator)
        for i, layer in enumerate(layers):
            if float(probs[i]) > drop_p:
                yield i, layer
    else:
        yield from enumerate(layers)


class StandardTransformerEncoder(TransformerEncoder):
    def __init__(self, layers: Iterable[TransformerEncoderLayer], layer_norm: LayerNorm | None = None, *,
                 layer_drop_p: float = 0.0) -> None:
        super().__init__()
        self.layers = ModuleList(layers)
        self.layer_norm = layer_norm
        self.layer_drop_p = layer_drop_p
        #: source of the LayerDrop decisions (``None``: the global CPU generator, which jobs seed differently on
        #: every rank). A data-parallel engine whose collectives need every rank to run the same layers installs a
        #: generator that is seeded identically everywhere.
        self.layer_drop_generator: torch.Generator | None = None

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> Tensor:
        cache = AttentionBiasCache()
        n = len(self.layers)
        for i, layer in drop_iter(self.layers, self.layer_drop_p, self.training, self.layer_drop_generator):
            seqs = layer(seqs, seqs_layout, cache)
            stop = False
            for hook in self._layer_hooks.values():
                if not hook(i, seqs, seqs_layout, n):  # type: ignore[operator]
                    stop = True
            if stop:
                break
        if self.layer_norm is not None:
            seqs = self.layer_norm(seqs)
        return seqs
