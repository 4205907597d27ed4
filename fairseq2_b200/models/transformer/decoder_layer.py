"""Transformer decoder layer with cross-attention (cf. fairseq2 ``models/transformer/decoder_layer.py:61-277``)."""
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


class TransformerDecoderLayer(Module, ABC):
    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, encoder_output: Tensor,
                encoder_output_layout: BatchLayout, self_attn_bias_cache: AttentionBiasCache,
                encoder_decoder_attn_bias_cache: AttentionBiasCache, *,
                state_bag: IncrementalStateBag | None = None) -> Tensor: ...


class StandardTransformerDecoderLayer(TransformerDecoderLayer):
    def __init__(self, self_attn: MultiheadAttention, self_attn_layer_norm: LayerNorm,
                 encoder_decoder_attn: MultiheadAttention, encoder_decoder_attn_layer_norm: LayerNorm,
                 ffn: FeedForwardNetwork, ffn_layer_norm: LayerNorm, *,
                 norm_order: TransformerNormOrder = TransformerNormOrder.POST, self_attn_norm: LayerNorm | None = None,
                 self_attn_residual: ResidualConnect | None = None,
                 encoder_decoder_attn_residual: ResidualConnect | None = None,
                 ffn_residual: ResidualConnect | None = None, dropout_p: float = 0.0) -> None:
        super().__init__()
        self.self_attn, self.self_attn_layer_norm, self.self_attn_norm = self_attn, self_attn_layer_norm, self_attn_norm
        self.encoder_decoder_attn = encoder_decoder_attn
        self.encoder_decoder_attn_layer_norm = encoder_decoder_attn_layer_norm
        self.ffn, self.ffn_layer_norm = ffn, ffn_layer_norm
        self.norm_order = norm_order
        self.self_attn_residual = self_attn_residual or AdditiveResidualConnect()
        self.encoder_decoder_attn_residual = encoder_decoder_attn_residual or AdditiveResidualConnect()
        self.ffn_residual = ffn_residual or AdditiveResidualConnect()
        mk = (lambda: Dropout(dropout_p)) if dropout_p > 0.0 else (lambda: None)
        self.self_attn_dropout, self.encoder_decoder_attn_dropout, self.ffn_dropout = mk(), mk(), mk()

    def forward(self, seqs, seqs_layout, encoder_output, encoder_output_layout, self_attn_bias_cache,  # type: ignore[override]
                encoder_decoder_attn_bias_cache, *, state_bag=None):
        pre = self.norm_order != TransformerNormOrder.POST
        # self attention
        residual = seqs
        if pre:
            seqs = self.self_attn_layer_norm(seqs)
        seqs = self.self_attn(seqs, seqs_layout, seqs, seqs_layout, seqs, self_attn_bias_cache, state_bag=state_bag)
        if self.self_attn_norm is not None:
            seqs = self.self_attn_norm(seqs)
        if self.self_attn_dropout is not None:
            seqs = self.self_attn_dropout(seqs)
        seqs = self.self_attn_residual(seqs, residual)
        if not pre:
            seqs = self.self_attn_layer_norm(seqs)
        # attention over the encoder output
        residual = seqs
        if pre:
            seqs = self.encoder_decoder_attn_layer_norm(seqs)
        seqs = self.encoder_decoder_attn(seqs, seqs_layout, encoder_output, encoder_output_layout, encoder_output,
                                         encoder_decoder_attn_bias_cache, state_bag=state_bag)
        if self.encoder_decoder_attn_dropout is not None:
            seqs = self.encoder_decoder_attn_dropout(seqs)
        seqs = self.encoder_decoder_attn_residual(seqs, residual)
        if not pre:
            seqs = self.encoder_decoder_attn_layer_norm(seqs)
        # feed-forward
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
