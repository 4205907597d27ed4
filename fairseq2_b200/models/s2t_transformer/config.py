"""S2T Transformer / Conformer configuration (cf. fairseq2 ``models/s2t_transformer/config.py:19-106``,
``models/s2t_conformer/config.py:18-70``)."""
from __future__ import annotations

from dataclasses import dataclass

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

S2T_TRANSFORMER_FAMILY = "s2t_transformer"
S2T_CONFORMER_FAMILY = "s2t_conformer"


@dataclass(kw_only=True)
class S2TTransformerConfig:
    """Defaults: the medium speech-to-text Transformer."""

    model_dim: int = 512
    max_source_seq_len: int = 1024
    num_fbank_channels: int = 80
    max_target_seq_len: int = 1024
    target_vocab_size: int = 10_000
    pad_idx: int = 1
    num_encoder_layers: int = 12
    num_decoder_layers: int = 6
    num_encoder_attn_heads: int = 8
    num_decoder_attn_heads: int = 8
    ffn_inner_dim: int = 512 * 4
    dropout_p: float = 0.15


@dataclass(kw_only=True)
class S2TConformerConfig:
    model_dim: int = 256
    max_source_seq_len: int = 6000
    num_fbank_channels: int = 80
    max_target_seq_len: int = 1024
    target_vocab_size: int = 181
    pad_idx: int = 1
    use_relative_pos: bool = False
    num_encoder_layers: int = 12
    num_decoder_layers: int = 6
    num_encoder_attn_heads: int = 4
    num_decoder_attn_heads: int = 8
    depthwise_conv_kernel_size: int = 31
    ffn_inner_dim: int = 512 * 4
    dropout_p: float = 0.1


arch = ConfigRegistrar(S2TTransformerConfig)
conformer_arch = ConfigRegistrar(S2TConformerConfig)


@arch("medium")
def medium() -> S2TTransformerConfig:
    return S2TTransformerConfig()


@arch("tiny")
def tiny() -> S2TTransformerConfig:
    return S2TTransformerConfig(model_dim=256, num_encoder_layers=6, num_decoder_layers=3, num_encoder_attn_heads=4,
                                num_decoder_attn_heads=4, ffn_inner_dim=256 * 4, dropout_p=0.3)


@arch("small")
def small() -> S2TTransformerConfig:
    return S2TTransformerConfig(model_dim=256, num_encoder_attn_heads=4, num_decoder_attn_heads=4,
                                ffn_inner_dim=256 * 8, dropout_p=0.1)


@arch("large")
def large() -> S2TTransformerConfig:
    return S2TTransformerConfig(model_dim=1024, num_encoder_attn_heads=16, num_decoder_attn_heads=16,
                                ffn_inner_dim=1024 * 4, dropout_p=0.2)


@conformer_arch("medium")
def conformer_medium() -> S2TConformerConfig:
    return S2TConformerConfig()


@conformer_arch("medium_rel_pos")
def conformer_medium_rel_pos() -> S2TConformerConfig:
    return S2TConformerConfig(use_relative_pos=True)
