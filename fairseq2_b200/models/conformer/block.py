"""Conformer block (cf. fairseq2 ``models/conformer/block.py:31-196``): half-step FFN, self-attention,
convolution module, half-step FFN and a closing layer norm, each with a pre-norm residual branch."""
from __future__ import annotations

from torch import Tensor
from torch.nn import Dropout

from fairseq2_b200.models.conformer.convolution import ConformerConvolution
from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer.encoder_layer import TransformerEncoderLayer
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.normalization import LayerNorm


class ConformerBlock(TransformerEncoderLayer):
    def __init__(self, ffn1_layer_norm: LayerNorm, ffn1: FeedForwardNetwork, self_attn_layer_norm: LayerNorm,
                 self_attn: MultiheadAttention, conv_layer_norm: LayerNorm, conv: ConformerConvolution,
                 ffn2_layer_norm: LayerNorm, ffn2: FeedForwardNetwork, layer_norm: LayerNorm, *,
                 dropout_p: float = 0.0) -> None:
        super().__init__()
        self.ffn1_layer_norm, self.ffn1 = ffn1_layer_norm, ffn1
        self.self_attn_layer_norm, self.self_attn = self_attn_layer_norm, self_attn
        self.conv_layer_norm, self.conv = conv_layer_norm, conv
        self.ffn2_layer_norm, self.ffn2 = ffn2_layer_norm, ffn2
        self.layer_norm = layer_norm
        mk = (lambda: Dropout(dropout_p)) if dropout_p > 0.0 else (lambda: None)
        self.ffn1_dropout, self.self_attn_dropout, self.conv_dropout, self.ffn2_dropout = mk(), mk(), mk(), mk()

    @staticmethod
    def _drop(d: Dropout | None, x: Tensor) -> Tensor:
        return d(x) if d is not None else x

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, bias_cache: AttentionBiasCache) -> Tensor:
        seqs = seqs + self._drop(self.ffn1_dropout, self.ffn1(self.ffn1_layer_norm(seqs)) * 0.5)
        x = self.self_attn_layer_norm(seqs)
        x = self.self_attn(x, seqs_layout, x, seqs_layout, x, bias_cache)
        seqs = seqs + self._drop(self.self_attn_dropout, x)
        seqs = seqs + self._drop(self.conv_dropout, self.conv(self.conv_layer_norm(seqs), seqs_layout))
        seqs = seqs + self._drop(self.ffn2_dropout, self.ffn2(self.ffn2_layer_norm(seqs)) * 0.5)
        return self.layer_norm(seqs)
