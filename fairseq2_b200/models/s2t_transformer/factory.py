"""Builds S2T Transformer and S2T Conformer models (cf. fairseq2 ``models/s2t_transformer/factory.py:49-265``,
``models/s2t_conformer/factory.py:54-320``)."""
from __future__ import annotations

import torch

from fairseq2_b200.models.conformer import ConformerBlock, ConformerConvolution
from fairseq2_b200.models.s2t_transformer.config import S2TConformerConfig, S2TTransformerConfig
from fairseq2_b200.models.s2t_transformer.frontend import Conv1dFbankSubsampler, S2TTransformerFrontend
from fairseq2_b200.models.transformer.attention_bias import CausalAttentionBias, IdentityBias
from fairseq2_b200.models.transformer.decoder import StandardTransformerDecoder
from fairseq2_b200.models.transformer.decoder_layer import StandardTransformerDecoderLayer
from fairseq2_b200.models.transformer.encoder import StandardTransformerEncoder
from fairseq2_b200.models.transformer.encoder_layer import StandardTransformerEncoderLayer
from fairseq2_b200.models.transformer.ffn import StandardFeedForwardNetwork
from fairseq2_b200.models.transformer.frontend import TransformerEmbeddingFrontend
from fairseq2_b200.models.transformer.model import TransformerModel
from fairseq2_b200.models.transformer.multihead_attention import StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import SDPA, create_default_sdpa
from fairseq2_b200.models.transformer.sdpa_relative import RelativePositionalEncoding, RelativePositionSDPA
from fairseq2_b200.nn.embedding import StandardEmbedding, init_scaled_embedding
from fairseq2_b200.nn.normalization import StandardLayerNorm
from fairseq2_b200.nn.position_encoder import SinusoidalPositionEncoder
from fairseq2_b200.nn.projection import Linear


def _init_final_projection(p: Linear) -> None:
    torch.nn.init.normal_(p.weight, std=p.weight.shape[1] ** -0.5)
    if p.bias is not None:
        torch.nn.init.zeros_(p.bias)


def _decoder(c: S2TTransformerConfig | S2TConformerConfig):  # type: ignore[no-untyped-def]
    embed = StandardEmbedding(c.target_vocab_size, c.model_dim, c.pad_idx, init_fn=init_scaled_embedding)
    pe = SinusoidalPositionEncoder(c.model_dim, c.max_target_seq_len, _legacy_pad_idx=1)
    frontend = TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=pe, dropout_p=c.dropout_p)

    def norm() -> StandardLayerNorm:
        return StandardLayerNorm(c.model_dim, bias=True)

    layers = []
    for _ in range(c.num_decoder_layers):
        sa = StandardMultiheadAttention(c.model_dim, c.num_decoder_attn_heads,
                                        create_default_sdpa(CausalAttentionBias(), dropout_p=c.dropout_p))
        ca = StandardMultiheadAttention(c.model_dim, c.num_decoder_attn_heads,
                                        create_default_sdpa(IdentityBias(), dropout_p=c.dropout_p))
        ffn = StandardFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=True)
        layers.append(StandardTransformerDecoderLayer(sa, norm(), ca, norm(), ffn, norm(),
                                                      norm_order=TransformerNormOrder.PRE, dropout_p=c.dropout_p))
    final = Linear(c.model_dim, c.target_vocab_size, bias=False, init_fn=_init_final_projection)
    return frontend, StandardTransformerDecoder(layers, norm()), final


def create_s2t_transformer_model(config: S2TTransformerConfig, gangs: object | None = None) -> TransformerModel:
    c = config
    sub = Conv1dFbankSubsampler(c.num_fbank_channels, 1024, c.model_dim, kernel_sizes=[5, 5])
    pe = SinusoidalPositionEncoder(c.model_dim, c.max_source_seq_len, _legacy_pad_idx=1)
    enc_frontend = S2TTransformerFrontend(c.model_dim, sub, pe, proj=None, dropout_p=c.dropout_p)

    def norm() -> StandardLayerNorm:
        return StandardLayerNorm(c.model_dim, bias=True)

    layers = []
    for _ in range(c.num_encoder_layers):
        sa = StandardMultiheadAttention(c.model_dim, c.num_encoder_attn_heads,
                                        create_default_sdpa(IdentityBias(), dropout_p=c.dropout_p))
        ffn = StandardFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=True)
        layers.append(StandardTransformerEncoderLayer(sa, norm(), ffn, norm(), norm_order=TransformerNormOrder.PRE,
                                                      dropout_p=c.dropout_p))
    dec_frontend, decoder, final = _decoder(c)
    return TransformerModel(c.model_dim, enc_frontend, StandardTransformerEncoder(layers, norm()), dec_frontend,
                            decoder, final, c.pad_idx, c.max_source_seq_len, c.max_target_seq_len)


def create_s2t_conformer_model(config: S2TConformerConfig, gangs: object | None = None) -> TransformerModel:
    c = config
    sub = Conv1dFbankSubsampler(c.num_fbank_channels, 1024, c.model_dim, kernel_sizes=[5, 5])
    pe = None if c.use_relative_pos else SinusoidalPositionEncoder(c.model_dim, c.max_source_seq_len, _legacy_pad_idx=1)
    enc_frontend = S2TTransformerFrontend(c.model_dim, sub, pe, proj=Linear(c.model_dim, c.model_dim, bias=True),
                                          dropout_p=c.dropout_p)
    rel = RelativePositionalEncoding(c.model_dim, c.max_source_seq_len) if c.use_relative_pos else None

    def norm() -> StandardLayerNorm:
        return StandardLayerNorm(c.model_dim, bias=True)

    def ffn() -> StandardFeedForwardNetwork:
        return StandardFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=True, inner_activation=torch.nn.SiLU(),
                                          inner_dropout_p=c.dropout_p)

    blocks = []
    for _ in range(c.num_encoder_layers):
        sdpa: SDPA
        if rel is not None:
            sdpa = RelativePositionSDPA(c.model_dim, c.num_encoder_attn_heads, rel, IdentityBias())
        else:
            sdpa = create_default_sdpa(IdentityBias(), dropout_p=c.dropout_p)
        sa = StandardMultiheadAttention(c.model_dim, c.num_encoder_attn_heads, sdpa)
        conv = ConformerConvolution(c.model_dim, c.depthwise_conv_kernel_size)
        blocks.append(ConformerBlock(norm(), ffn(), norm(), sa, norm(), conv, norm(), ffn(), norm(),
                                     dropout_p=c.dropout_p))
    dec_frontend, decoder, final = _decoder(c)
    return TransformerModel(c.model_dim, enc_frontend, StandardTransformerEncoder(blocks, None), dec_frontend,
                            decoder, final, c.pad_idx, c.max_source_seq_len, c.max_target_seq_len)
