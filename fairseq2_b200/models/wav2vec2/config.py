"""wav2vec 2.0 configuration (cf. fairseq2 ``models/wav2vec2/config.py:22-234``)."""
from __future__ import annotations

from dataclasses import dataclass, field

from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.runtime.config_registry import ConfigRegistrar
from fairseq2_b200.utils.validation import ValidationResult

WAV2VEC2_FAMILY = "wav2vec2"


def _default_descs() -> list[tuple[int, int, int]]:
    return [(512, 10, 5)] + [(512, 3, 2)] * 4 + [(512, 2, 2)] * 2


@dataclass(kw_only=True)
class Wav2Vec2EncoderConfig:
    model_dim: int = 768
    max_seq_len: int = 4096
    feature_dim: int = 512
    use_fbank: bool = False
    first_pass_dropout_p: float = 0.0
    layer_norm_features: bool = True
    feature_extractor_layer_descs: list[tuple[int, int, int]] = field(default_factory=_default_descs)
    feature_extractor_bias: bool = False
    feature_extractor_layer_norm_convs: bool = False
    feature_grad_scale: float = 0.1
    num_fbank_channels: int = 0
    fbank_stride: int = 0
    sample_fbank_every_k: int = 0
    pos_encoder_type: str = "conv"
    """``conv``, ``relative`` or ``rotary``."""
    pos_encoder_depth: int = 1
    pos_conv_kernel_size: int = 128
    num_pos_conv_groups: int = 16
    use_conformer: bool = False
    num_encoder_layers: int = 12
    num_encoder_attn_heads: int = 12
    ffn_inner_dim: int = 3072
    dropout_p: float = 0.1
    attn_dropout_p: float = 0.1
    ffn_inner_dropout_p: float = 0.0
    layer_drop_p: float = 0.05
    norm_order: TransformerNormOrder = TransformerNormOrder.POST
    depthwise_conv_kernel_size: int = 0

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        if self.use_conformer and self.norm_order != TransformerNormOrder.POST:
            r.add_error(f"`norm_order` must be `POST` when `use_conformer` is `True`, but is `{self.norm_order}`.")
        return r


@dataclass(kw_only=True)
class Wav2Vec2Config:
    encoder_config: Wav2Vec2EncoderConfig = field(default_factory=Wav2Vec2EncoderConfig)
    final_dim: int = 256
    final_proj_bias: bool = True
    quantizer_encoder_grad: bool = True
    temporal_mask_span_len: int = 10
    max_temporal_mask_prob: float = 0.69
    min_num_temporal_mask_spans: int = 2
    spatial_mask_span_len: int = 10
    max_spatial_mask_prob: float = 0.0
    min_num_spatial_mask_spans: int = 2
    quantized_dim: int = 256
    num_codebooks: int = 2
    num_codebook_entries: int = 320
    codebook_sampling_temperature: tuple[float, float, float] = (2.0, 0.5, 0.999995)
    num_distractors: int = 100
    logit_temp: float = 0.1


arch = ConfigRegistrar(Wav2Vec2Config)
encoder_arch = ConfigRegistrar(Wav2Vec2EncoderConfig)


@arch("base")
def base() -> Wav2Vec2Config:
    return Wav2Vec2Config()


@arch("large")
def large() -> Wav2Vec2Config:
    c = base()
    e = c.encoder_config
    e.model_dim, e.num_encoder_layers, e.num_encoder_attn_heads, e.ffn_inner_dim = 1024, 24, 16, 4096
    e.dropout_p, e.layer_drop_p = 0.0, 0.2
    c.quantized_dim = c.final_dim = 768
    return c


@arch("large_lv60k")
def large_lv60k() -> Wav2Vec2Config:
    c = large()
    e = c.encoder_config
    e.layer_norm_features = False
    e.feature_extractor_bias = True
    e.feature_extractor_layer_norm_convs = True
    e.layer_drop_p = 0.0
    e.norm_order = TransformerNormOrder.PRE
    c.codebook_sampling_temperature = (2.0, 0.1, 0.999995)
    return c


@arch("xlsr_base")
def xlsr_base() -> Wav2Vec2Config:
    c = large_lv60k()
    c.encoder_config.attn_dropout_p = 0.0
    c.encoder_config.feature_grad_scale = 1.0
    c.quantized_dim = c.final_dim = 1024
    return c


@arch("tiny")
def tiny() -> Wav2Vec2Config:
    e = Wav2Vec2EncoderConfig(model_dim=64, max_seq_len=512, feature_dim=32,
                              feature_extractor_layer_descs=[(32, 10, 5), (32, 3, 2), (32, 2, 2)],
                              pos_conv_kernel_size=16, num_pos_conv_groups=4, num_encoder_layers=2,
                              num_encoder_attn_heads=4, ffn_inner_dim=128, dropout_p=0.0, attn_dropout_p=0.0,
                              layer_drop_p=0.0)
    return Wav2Vec2Config(encoder_config=e, final_dim=32, quantized_dim=32, num_codebook_entries=16,
                          num_distractors=10, temporal_mask_span_len=3, min_num_temporal_mask_spans=2)


for _name, _fn in (("base", base), ("large", large), ("large_lv60k", large_lv60k), ("xlsr_base", xlsr_base),
                   ("tiny", tiny)):
    encoder_arch(_name)(lambda f=_fn: f().encoder_config)
