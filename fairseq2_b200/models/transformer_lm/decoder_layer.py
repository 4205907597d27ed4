"""Decoder-only transformer layer (cf. fairseq2 ``models/transformer_lm/decoder_layer.py:58-209``)."""
from __future__ import annotations

from abc import ABC, abstractmethod

from torch import Tensor
from torch.nn import Dropout, Module

from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm
from fairseq2_b200.nn.residual import AdditiveResidualConnect, ResidualConnect


class TransformerLMDecoderLayer(Module, ABC):
    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, bias_cache: AttentionBiasCache, *,
                state_bag: IncrementalStateBag | None = None) -> Tensor: ...


class StandardTransformerLMDecoderLayer(TransformerLMDecoderLayer):
    def __init__(self, self_attn: MultiheadAttention, self_attn_layer_norm: LayerNorm, ffn: FeedForwardNetwork,
                 ffn_layer_norm: LayerNorm, *, norm_order: TransformerNormOrder = TransformerNormOrder.POST,
                 self_attn_residual: ResidualConnect | None = None, ffn_residual: ResidualConnect | None = None,
                 dropout_p: float = 0.0) -> None:
        super().__init__()
        self.self_attn, self.self_attn_layer_norm = self_attn, self_attn_layer_norm
        self.ffn, self.ffn_layer_norm = ffn, ffn_layer_norm
        self.norm_order = norm_order
        self.self_attn_residual = self_attn_residual or AdditiveResidualConnect()
        self.ffn_residual = ffn_residual or AdditiveResidualConnect()
        self.self_attn_dropout = Dropout(dropout_p) if dropout_p > 0.0 else None
        self.ffn_dropout = Dropout(dropout_p) if dropout_p > 0.0 else None

    @property
    def supports_deferred_residual(self) -> bool:
        """True if both residual adds of this layer can be folded into the RMSNorm that follows them (pre-norm,
        plain additive residuals, no dropout, RMSNorm with a weight and no bias)."""
        from fairseq2_b200.nn.normalization import RMSNorm

        def plain_rms(n: LayerNorm) -> bool:
            return (type(n) is RMSNorm and n.weight is not None and n.bias is None and len(n.normalized_shape) == 1)

        return (self.norm_order == TransformerNormOrder.PRE and type(self.self_attn_residual) is AdditiveResidualConnect
                and type(self.ffn_residual) is AdditiveResidualConnect and self.self_attn_dropout is None
                and self.ffn_dropout is None and plain_rms(self.self_attn_layer_norm)
                and plain_rms(self.ffn_layer_norm))

    def _forward_deferred(self, seqs, seqs_layout, bias_cache, state_bag, delta):  # type: ignore[no-untyped-def]
        """The hidden state enters as ``seqs + delta`` (``delta`` = the previous layer's feed-forward output, not
        yet added) and leaves the same way, so that every residual add runs inside the norm kernel that consumes
        the sum: one pass over the activations instead of an add, a write and a re-read."""
        from fairseq2_b200.ops.norm import add_rms_norm

        n1, n2 = self.self_attn_layer_norm, self.ffn_layer_norm
        if delta is not None:
            residual, y = add_rms_norm(delta, seqs, n1.weight, n1.eps)
        else:
            residual, y = seqs, n1(seqs)
        attn = self.self_attn(y, seqs_layout, y, seqs_layout, y, bias_cache, state_bag=state_bag)
        hidden, y2 = add_rms_norm(attn, residual, n2.weight, n2.eps)
        return hidden, self.ffn(y2)

    def forward(self, seqs, seqs_layout, bias_cache, *, state_bag=None, delta=None,  # type: ignore[override]
                defer_residual=False):
        if defer_residual:
            return self._forward_deferred(seqs, seqs_layout, bias_cache, state_bag, delta)
        if delta is not None:
            seqs = seqs + delta
        pre = self.norm_order != TransformerNormOrder.POST
        residual = seqs
        if pre:
            seqs = self.self_attn_layer_norm(seqs)
        seqs = self.self_attn(seqs, seqs_layout, seqs, seqs_layout, seqs, bias_cache, state_bag=state_bag)
        if self.self_attn_dropout is not None:
            seqs = self.self_attn_dropout(seqs)
        seqs = self.self_attn_residual(seqs, residual)
        if not pre:
            seqs = self.self_attn_layer_norm(seqs)
        residual = seqs
        if pre:
            seqs = self.ffn_layer_norm(seqs)
        seqs = self.ffn(seqs)
        if self.ffn_dropout is not None:
            seqs = self.ffn_dropout(seqs)
        seqs = self.ffn_residual(seqs, residual)
        if not pre:
            seqs = self.ffn_layer_norm(seqs)
        return seqs
