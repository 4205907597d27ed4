"""Builds wav2vec 2.0 models and encoders (cf. fairseq2 ``models/wav2vec2/factory.py:58-354``)."""
from __future__ import annotations

import torch

from fairseq2_b200.models.conformer import ConformerBlock, ConformerConvolution
from fairseq2_b200.models.feature_extractor import SequenceFeatureExtractor
from fairseq2_b200.models.transformer.attention_bias import IdentityBias
from fairseq2_b200.models.transformer.encoder import StandardTransformerEncoder, TransformerEncoder
from fairseq2_b200.models.transformer.encoder_layer import StandardTransformerEncoderLayer, TransformerEncoderLayer
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork, StandardFeedForwardNetwork
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention, StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import SDPA, create_default_sdpa
from fairseq2_b200.models.transformer.sdpa_relative import RelativePositionalEncoding, RelativePositionSDPA
from fairseq2_b200.models.wav2vec2.config import Wav2Vec2Config, Wav2Vec2EncoderConfig
from fairseq2_b200.models.wav2vec2.feature_extractor import Wav2Vec2FbankFeatureExtractor, Wav2Vec2FeatureExtractor
from fairseq2_b200.models.wav2vec2.frontend import Wav2Vec2Frontend
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker
from fairseq2_b200.models.wav2vec2.model import Wav2Vec2Model
from fairseq2_b200.models.wav2vec2.position_encoder import Wav2Vec2PositionEncoder, Wav2Vec2StackedPositionEncoder
from fairseq2_b200.models.wav2vec2.vector_quantizer import GumbelVectorQuantizer, VectorQuantizer
from fairseq2_b200.nn.normalization import LayerNorm, StandardLayerNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder, RotaryEncoder
from fairseq2_b200.nn.projection import Linear


def create_wav2vec2_model(config: Wav2Vec2Config, gangs: object | None = None) -> Wav2Vec2Model:
    return Wav2Vec2Factory(config).create_model()


def init_bert_projection(p: Linear) -> None:
    """BERT-style initialisation used by the wav2vec 2.0 encoder."""
    torch.nn.init.normal_(p.weight, mean=0.0, std=0.02)
    if p.bias is not None:
        torch.nn.init.zeros_(p.bias)


class Wav2Vec2Factory:
    def __init__(self, config: Wav2Vec2Config) -> None:
        self._config = config

    def create_model(self) -> Wav2Vec2Model:
        c = self._config
        ef = Wav2Vec2EncoderFactory(c.encoder_config)
        frontend, encoder = ef.create_encoder_frontend(), ef.create_encoder()
        return Wav2Vec2Model(c.encoder_config.model_dim, frontend, encoder, self.create_masker(),
                             self.create_quantizer(), c.final_dim, final_proj_bias=c.final_proj_bias,
                             num_distractors=c.num_distractors, logit_temp=c.logit_temp,
                             quantizer_encoder_grad=c.quantizer_encoder_grad)

    def create_masker(self) -> Wav2Vec2Masker:
        c = self._config
        return Wav2Vec2Masker(c.encoder_config.model_dim, c.temporal_mask_span_len, c.max_temporal_mask_prob,
                              c.min_num_temporal_mask_spans, c.spatial_mask_span_len, c.max_spatial_mask_prob,
                              c.min_num_spatial_mask_spans)

    def create_quantizer(self) -> VectorQuantizer:
        c = self._config
        return GumbelVectorQuantizer(c.encoder_config.feature_dim, c.quantized_dim, c.num_codebooks,
                                     c.num_codebook_entries,
                                     codebook_sampling_temperature=c.codebook_sampling_temperature)


class Wav2Vec2EncoderFactory:
    def __init__(self, config: Wav2Vec2EncoderConfig) -> None:
        self._config = config
        self._rel_pos: RelativePositionalEncoding | None = None

    def create_encoder_frontend(self) -> Wav2Vec2Frontend:
        c = self._config
        return Wav2Vec2Frontend(c.model_dim, c.feature_dim, self.create_feature_extractor(),
                                self.create_position_encoder(), first_pass_dropout_p=c.first_pass_dropout_p,
                                layer_norm=c.norm_order == TransformerNormOrder.POST, dropout_p=c.dropout_p)

    def create_feature_extractor(self) -> SequenceFeatureExtractor:
        c = self._config
        if c.use_fbank:
            return Wav2Vec2FbankFeatureExtractor(c.num_fbank_channels, c.fbank_stride,
                                                 sample_every_k=c.sample_fbank_every_k)
        return Wav2Vec2FeatureExtractor(c.feature_extractor_layer_descs, c.feature_extractor_bias,
                                        layer_norm=c.feature_extractor_layer_norm_convs,
                                        grad_scale=c.feature_grad_scale)

    def create_position_encoder(self) -> PositionEncoder | None:
        c = self._config
        if c.pos_encoder_type != "conv":
            return None
        if c.pos_encoder_depth == 1:
            return Wav2Vec2PositionEncoder(c.model_dim, c.pos_conv_kernel_size, c.num_pos_conv_groups)
        return Wav2Vec2StackedPositionEncoder(c.model_dim, c.pos_conv_kernel_size, c.num_pos_conv_groups,
                                              c.pos_encoder_depth)

    def create_encoder(self) -> TransformerEncoder:
        c = self._config
        mk = self.create_conformer_block if c.use_conformer else self.create_encoder_layer
        layers = [mk() for _ in range(c.num_encoder_layers)]
        norm = self.create_layer_norm() if (not c.use_conformer and c.norm_order != TransformerNormOrder.POST) else None
        return StandardTransformerEncoder(layers, norm, layer_drop_p=c.layer_drop_p)

    def create_encoder_layer(self) -> TransformerEncoderLayer:
        c = self._config
        return StandardTransformerEncoderLayer(self.create_self_attention(), self.create_layer_norm(),
                                               self.create_ffn(), self.create_layer_norm(), norm_order=c.norm_order,
                                               dropout_p=c.dropout_p)

    def create_conformer_block(self) -> TransformerEncoderLayer:
        c = self._config
        conv = ConformerConvolution(c.model_dim, c.depthwise_conv_kernel_size)
        return ConformerBlock(self.create_layer_norm(), self.create_ffn(use_swish=True), self.create_layer_norm(),
                              self.create_self_attention(), self.create_layer_norm(), conv, self.create_layer_norm(),
                              self.create_ffn(use_swish=True), self.create_layer_norm(), dropout_p=c.dropout_p)

    def create_self_attention(self) -> MultiheadAttention:
        c = self._config
        pos = None
        if c.pos_encoder_type == "rotary":
            pos = RotaryEncoder(c.model_dim // c.num_encoder_attn_heads, c.max_seq_len)
        sdpa: SDPA
        if c.pos_encoder_type == "relative":
            if self._rel_pos is None:
                self._rel_pos = RelativePositionalEncoding(c.model_dim, c.max_seq_len)   # shared by every layer
            sdpa = RelativePositionSDPA(c.model_dim, c.num_encoder_attn_heads, self._rel_pos, IdentityBias())
        else:
            sdpa = create_default_sdpa(IdentityBias(), dropout_p=c.attn_dropout_p)
        return StandardMultiheadAttention(c.model_dim, c.num_encoder_attn_heads, sdpa, pos_encoder=pos,
                                          qkv_proj_init_fn=init_bert_projection,
                                          output_proj_init_fn=init_bert_projection)

    def create_ffn(self, use_swish: bool = False) -> FeedForwardNetwork:
        c = self._config
        return StandardFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=True,
                                          inner_activation=torch.nn.SiLU() if use_swish else torch.nn.GELU(),
                                          inner_dropout_p=c.ffn_inner_dropout_p,
                                          proj_init_fn=init_bert_projection)

    def create_layer_norm(self) -> LayerNorm:
        return StandardLayerNorm(self._config.model_dim, bias=True)
