"""Builds NLLB translation models (cf. fairseq2 ``models/nllb/factory.py:47-245``): pre-norm encoder-decoder
Transformer with a shared, scaled embedding table, sinusoidal positions and a tied output projection."""
from __future__ import annotations

from fairseq2_b200.models.nllb.config import NllbConfig
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
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.nn.embedding import StandardEmbedding, init_scaled_embedding
from fairseq2_b200.nn.normalization import StandardLayerNorm
from fairseq2_b200.nn.position_encoder import SinusoidalPositionEncoder
from fairseq2_b200.nn.projection import TiedProjection


def create_nllb_model(config: NllbConfig, gangs: object | None = None) -> TransformerModel:
    c = config
    embed = StandardEmbedding(c.vocab_size, c.model_dim, c.pad_idx, init_fn=init_scaled_embedding)

    def frontend() -> TransformerEmbeddingFrontend:
        pe = SinusoidalPositionEncoder(c.model_dim, c.max_seq_len, _legacy_pad_idx=1)
        return TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=pe, dropout_p=c.dropout_p)

    def norm() -> StandardLayerNorm:
        return StandardLayerNorm(c.model_dim, bias=True)

    def attn(heads: int, causal: bool) -> StandardMultiheadAttention:
        bias = CausalAttentionBias() if causal else IdentityBias()
        return StandardMultiheadAttention(c.model_dim, heads, create_default_sdpa(bias))

    def ffn() -> StandardFeedForwardNetwork:
        return StandardFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=True)

    enc_layers = [StandardTransformerEncoderLayer(attn(c.num_encoder_attn_heads, False), norm(), ffn(), norm(),
                                                  norm_order=TransformerNormOrder.PRE, dropout_p=c.dropout_p)
                  for _ in range(c.num_encoder_layers)]
    dec_layers = [StandardTransformerDecoderLayer(attn(c.num_decoder_attn_heads, True), norm(),
                                                  attn(c.num_decoder_attn_heads, False), norm(), ffn(), norm(),
                                                  norm_order=TransformerNormOrder.PRE, dropout_p=c.dropout_p)
                  for _ in range(c.num_decoder_layers)]
    return TransformerModel(c.model_dim, frontend(), StandardTransformerEncoder(enc_layers, norm()), frontend(),
                            StandardTransformerDecoder(dec_layers, norm()), TiedProjection(embed.weight, bias=None),
                            c.pad_idx, c.max_seq_len, c.max_seq_len)
