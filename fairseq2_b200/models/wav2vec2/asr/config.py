"""wav2vec 2.0 ASR configuration (cf. fairseq2 ``models/wav2vec2/asr/config.py:24-135``)."""
from __future__ import annotations

from dataclasses import dataclass, field

from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.wav2vec2.config import Wav2Vec2EncoderConfig
from fairseq2_b200.runtime.config_registry import ConfigRegistrar

WAV2VEC2_ASR_FAMILY = "wav2vec2_asr"


def _base_10h_encoder() -> Wav2Vec2EncoderConfig:
    return Wav2Vec2EncoderConfig(feature_grad_scale=1.0, dropout_p=0.0, attn_dropout_p=0.0, ffn_inner_dropout_p=0.1)


@dataclass(kw_only=True)
class Wav2Vec2AsrConfig:
    """Defaults: the base model fine-tuned on 10 hours of Librispeech."""

    encoder_config: Wav2Vec2EncoderConfig = field(default_factory=_base_10h_encoder)
    target_vocab_size: int = 32
    final_dropout_p: float = 0.0
    use_masking: bool = True
    temporal_mask_span_len: int = 10
    max_temporal_mask_prob: float = 0.69
    min_num_temporal_mask_spans: int = 2
    spatial_mask_span_len: int = 64
    max_spatial_mask_prob: float = 0.55
    min_num_spatial_mask_spans: int = 2


arch = ConfigRegistrar(Wav2Vec2AsrConfig)


@arch("base_10h")
def base_10h() -> Wav2Vec2AsrConfig:
    return Wav2Vec2AsrConfig()


@arch("base_100h")
def base_100h() -> Wav2Vec2AsrConfig:
    c = base_10h()
    c.encoder_config.layer_drop_p = 0.1
    return c


@arch("large_10h")
def large_10h() -> Wav2Vec2AsrConfig:
    c = base_10h()
    e = c.encoder_config
    e.model_dim, e.num_encoder_layers, e.num_encoder_attn_heads, e.ffn_inner_dim = 1024, 24, 16, 4096
    e.layer_drop_p = 0.1
    c.max_temporal_mask_prob = 0.80
    c.max_spatial_mask_prob = 0.30
    return c


@arch("large_100h")
def large_100h() -> Wav2Vec2AsrConfig:
    c = large_10h()
    c.max_temporal_mask_prob = 0.53
    c.max_spatial_mask_prob = 0.55
    return c


@arch("large_lv60k_10h")
def large_lv60k_10h() -> Wav2Vec2AsrConfig:
    c = large_10h()
    e = c.encoder_config
    e.layer_norm_features = False
    e.feature_extractor_bias = True
    e.feature_extractor_layer_norm_convs = True
    e.norm_order = TransformerNormOrder.PRE
    c.max_spatial_mask_prob = 0.25
    return c


@arch("large_lv60k_100h")
def large_lv60k_100h() -> Wav2Vec2AsrConfig:
    c = large_lv60k_10h()
    c.max_temporal_mask_prob = 0.53
    return c


@arch("tiny")
def asr_tiny() -> Wav2Vec2AsrConfig:
    from fairseq2_b200.models.wav2vec2.config import tiny

    e = tiny().encoder_config
    e.feature_grad_scale = 1.0
    return Wav2Vec2AsrConfig(encoder_config=e, target_vocab_size=16, temporal_mask_span_len=3,
                             spatial_mask_span_len=8, max_spatial_mask_prob=0.2)
