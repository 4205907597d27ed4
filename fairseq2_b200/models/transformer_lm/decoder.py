"""Stack of decoder-only layers (cf. fairseq2 ``models/transformer_lm/decoder.py:101-160``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Iterable, Protocol

from torch import Tensor
from torch.nn import Module, ModuleList

from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer_lm.decoder_layer import TransformerLMDecoderLayer
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm


class TransformerLMDecoderLayerHook(Protocol):
    def __call__(self, layer_idx: int, layer_output: Tensor, layer_output_layout: BatchLayout,
                 num_layers: int) -> bool:
        """Return ``False`` to stop after this layer."""


class TransformerLMDecoder(Module, ABC):
    def __init__(self) -> None:
        super().__init__()
        self._layer_hooks: dict[int, TransformerLMDecoderLayerHook] = {}

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None
                ) -> Tensor: ...

    def register_layer_hook(self, hook: TransformerLMDecoderLayerHook):  # type: ignore[no-untyped-def]
        key = max(self._layer_hooks, default=-1) + 1
        self._layer_hooks[key] = hook
        hooks = self._layer_hooks

        class _Handle:
            def remove(self) -> None:
                hooks.pop(key, None)

        return _Handle()


class StandardTransformerLMDecoder(TransformerLMDecoder):
    def __init__(self, layers: Iterable[TransformerLMDecoderLayer], layer_norm: LayerNorm | None) -> None:
        super().__init__()
        self.layers = ModuleList(layers)
        self.layer_norm = layer_norm

    def _can_defer_residuals(self) -> bool:
        return (not self._layer_hooks and len(self.layers) > 0
                and all(getattr(layer, "supports_deferred_residual", False) for layer in self.layers))

    def forward(self, seqs, seqs_layout, *, state_bag=None):  # type: ignore[override]
        cache = AttentionBiasCache()
        n = len(self.layers)
        if self._can_defer_residuals():
            # every residual add is folded into the norm kernel that reads the sum (the next layer's first norm,
            # or the final norm below)
            from fairseq2_b200.nn.normalization import RMSNorm
            from fairseq2_b200.ops.norm import add_rms_norm

            delta = None
            for layer in self.layers:
                seqs, delta = layer(seqs, seqs_layout, cache, state_bag=state_bag, delta=delta, defer_residual=True)
            ln = self.layer_norm
            if type(ln) is RMSNorm and ln.weight is not None and ln.bias is None and len(ln.normalized_shape) == 1:
                return add_rms_norm(delta, seqs, ln.weight, ln.eps)[1]
            seqs = seqs + delta
            return ln(seqs) if ln is not None else seqs
        for i, layer in enumerate(self.layers):
            seqs = layer(seqs, seqs_layout, cache, state_bag=state_bag)
            stop = False
            for hook in self._layer_hooks.values():
                if not hook(i, seqs, seqs_layout, n):
                    stop = True
            if stop:
                break
        if self.layer_norm is not None:
            seqs = self.layer_norm(seqs)
        return seqs
