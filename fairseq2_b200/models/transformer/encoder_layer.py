"""Transformer encoder layer (cf. fairseq2 ``models/transformer/encoder_layer.py:54-203``)."""
from __future__ import annotations

from abc import ABC, abstractmethod

from torch import Tensor
from torch.nn import Dropout, Module

from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.normalization import LayerNorm
from fairseq2_b200.nn.residual import AdditiveResidualConnect, ResidualConnect


class TransformerEncoderLayer(Module, ABC):
    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, bias_cache: AttentionBiasCache) -> Tensor: ...


class StandardTransformerEncoderLayer(TransformerEncoderLayer):
    """Self-attention + FFN with POST, PRE or PRE_WITH_NORMFORMER ordering; the
    NormFormer variant takes the extra ``self_attn_norm`` applied to the attention output."""

    def __init__(self, self_attn: MultiheadAttention, self_attn_layer_norm: LayerNorm, ffn: FeedForwardNetwork,
                 ffn_layer_norm: LayerNorm, *, norm_order: TransformerNormOrder = TransformerNormOrder.POST,
                 self_attn_norm: LayerNorm | None = None, self_attn_residual: ResidualConnect | None = None,
                 ffn_residual: ResidualConnect | None = None, dropout_p: float = 0.0) -> None:
        super().__init__()
        self.self_attn, self.self_attn_layer_norm = self_attn, self_attn_layer_norm
        self.self_attn_norm = self_attn_norm
        self.ffn, self.ffn_layer_norm = ffn, ffn_layer_norm
        self.norm_order = norm_order
        self.self_attn_residual = self_attn_residual or AdditiveResidualConnect()
        self.ffn_residual = ffn_residual or AdditiveResidualConnect()
        self.self_attn_dropout = Dropout(dropout_p) if dropout_p > 0.0 else None
        self.ffn_dropout = Dropout(dropout_p) if dropout_p > 0.0 else None

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, bias_cache: AttentionBiasCache) -> Tensor:
        pre = self.norm_order != TransformerNormOrder.POST
        residual = seqs
        if pre:
            seqs = self.self_attn_layer_norm(seqs)
        seqs = self.self_attn(seqs, seqs_layout, seqs, seqs_layout, seqs, bias_cache)
        if self.self_attn_norm is not None:
            seqs = self.self_attn_norm(seqs)
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
