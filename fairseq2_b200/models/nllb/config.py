"""NLLB configuration (cf. fairseq2 ``models/nllb/config.py:19-87``)."""
from __future__ import annotations

from dataclasses import dataclass

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

NLLB_FAMILY = "nllb"


@dataclass(kw_only=True)
class NllbConfig:
    model_dim: int = 1024
    max_seq_len: int = 1024
    vocab_size: int = 256_206
    pad_idx: int = 0
    num_encoder_layers: int = 24
    num_decoder_layers: int = 24
    num_encoder_attn_heads: int = 16
    num_decoder_attn_heads: int = 16
    ffn_inner_dim: int = 1024 * 8
    dropout_p: float = 0.1


arch = ConfigRegistrar(NllbConfig)


@arch("dense_1b")
def dense_1b() -> NllbConfig:
    return NllbConfig()


@arch("dense_300m")
def dense_300m() -> NllbConfig:
    return NllbConfig(num_encoder_layers=6, num_decoder_layers=6, ffn_inner_dim=1024 * 4, dropout_p=0.3)


@arch("dense_600m")
def dense_600m() -> NllbConfig:
    return NllbConfig(num_encoder_layers=12, num_decoder_layers=12, ffn_inner_dim=1024 * 4)


@arch("dense_3b")
def dense_3b() -> NllbConfig:
    return NllbConfig(model_dim=2048)


@arch("tiny")
def nllb_tiny() -> NllbConfig:
    return NllbConfig(model_dim=64, max_seq_len=128, vocab_size=200, num_encoder_layers=2, num_decoder_layers=2,
                      num_encoder_attn_heads=4, num_decoder_attn_heads=4, ffn_inner_dim=128, dropout_p=0.0)
