"""Qwen 2.5 / Qwen 3 configuration (cf. fairseq2 ``models/qwen/config.py:19-330``)."""
from __future__ import annotations

from dataclasses import dataclass

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

QWEN_FAMILY = "qwen"


@dataclass(kw_only=True)
class QwenConfig:
    model_dim: int = 3584
    max_seq_len: int = 32_768
    vocab_size: int = 152_064
    tied_embeddings: bool = False
    num_layers: int = 28
    num_attn_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: int | None = None
    """``None``: ``model_dim // num_attn_heads``."""
    qkv_proj_bias: bool = True
    q_norm: bool = False
    k_norm: bool = False
    ffn_inner_dim: int = 18_944
    rope_theta: float = 1_000_000.0
    dropout_p: float = 0.0


arch = ConfigRegistrar(QwenConfig)


def _q25(name: str, **kw: object) -> None:
    @arch(name)
    def _f() -> QwenConfig:
        return QwenConfig(**kw)  # type: ignore[arg-type]


def _q3(name: str, **kw: object) -> None:
    @arch(name)
    def _f() -> QwenConfig:
        return QwenConfig(max_seq_len=40_960, vocab_size=151_936, head_dim=128, qkv_proj_bias=False, q_norm=True,
                          k_norm=True, **kw)  # type: ignore[arg-type]


_q25("qwen25_1_5b", model_dim=1536, vocab_size=151_936, tied_embeddings=True, num_attn_heads=12,
     num_key_value_heads=2, ffn_inner_dim=8960)
_q25("qwen25_3b", model_dim=2048, vocab_size=151_936, num_layers=36, num_attn_heads=16, num_key_value_heads=2,
     ffn_inner_dim=11_008, tied_embeddings=True)
_q25("qwen25_7b")
_q25("qwen25_14b", model_dim=5120, num_layers=48, num_attn_heads=40, num_key_value_heads=8, ffn_inner_dim=13_824)
_q25("qwen25_32b", model_dim=5120, num_layers=64, num_attn_heads=40, num_key_value_heads=8, ffn_inner_dim=27_648)
_q3("qwen3_0.6b", model_dim=1024, tied_embeddings=True, num_layers=28, num_attn_heads=16, num_key_value_heads=8,
    ffn_inner_dim=3072)
_q3("qwen3_1.7b", model_dim=2048, tied_embeddings=True, num_layers=28, num_attn_heads=16, num_key_value_heads=8,
    ffn_inner_dim=6144)
_q3("qwen3_4b", model_dim=2560, tied_embeddings=True, num_layers=36, num_attn_heads=32, num_key_value_heads=8,
    ffn_inner_dim=9728)
_q3("qwen3_8b", model_dim=4096, num_layers=36, num_attn_heads=32, num_key_value_heads=8, ffn_inner_dim=12_288)
_q3("qwen3_14b", model_dim=5120, num_layers=40, num_attn_heads=40, num_key_value_heads=8, ffn_inner_dim=17_408)
_q3("qwen3_32b", model_dim=5120, num_layers=64, num_attn_heads=64, num_key_value_heads=8, ffn_inner_dim=25_600)


@arch("tiny")
def qwen_tiny() -> QwenConfig:
    return QwenConfig(model_dim=128, max_seq_len=256, vocab_size=512, tied_embeddings=True, num_layers=2,
                      num_attn_heads=4, num_key_value_heads=2, head_dim=64, qkv_proj_bias=False, q_norm=True,
                      k_norm=True, ffn_inner_dim=256)
