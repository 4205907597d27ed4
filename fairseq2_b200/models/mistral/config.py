"""Mistral configuration (cf. fairseq2 ``models/mistral/config.py:19-67``)."""
from __future__ import annotations

from dataclasses import dataclass

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

MISTRAL_FAMILY = "mistral"


@dataclass(kw_only=True)
class MistralConfig:
    model_dim: int = 4096
    max_seq_len: int = 8192
    vocab_size: int = 32_000
    pad_idx: int | None = None
    attn_window_len: int = 4096
    """Sliding attention window; every position sees at most this many keys."""
    num_layers: int = 32
    num_attn_heads: int = 32
    num_key_value_heads: int = 8
    ffn_inner_dim: int = 14336
    rope_theta: float = 10_000.0
    dropout_p: float = 0.0


arch = ConfigRegistrar(MistralConfig)


@arch("7b")
def mistral_7b() -> MistralConfig:
    return MistralConfig()


@arch("tiny")
def mistral_tiny() -> MistralConfig:
    return MistralConfig(model_dim=128, max_seq_len=256, vocab_size=512, attn_window_len=16, num_layers=2,
                         num_attn_heads=4, num_key_value_heads=2, ffn_inner_dim=256)
