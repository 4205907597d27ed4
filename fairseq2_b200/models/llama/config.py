"""LLaMA family configuration and presets (cf. fairseq2 ``models/llama/config.py:18-272``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

from fairseq2_b200.runtime.config_registry import ConfigRegistrar, get_config_registry

LLAMA_FAMILY = "llama"


@dataclass
class LLaMARoPEScaleConfig:
    """LLaMA-3.1 long-context frequency smoothing."""

    factor: float = 8.0
    frequency_factors: tuple[float, float] = (1.0, 4.0)
    original_context_length: int = 8192


@dataclass(kw_only=True)
class LLaMAConfig:
    model_dim: int = 4096
    max_seq_len: int = 2048
    vocab_size: int = 32_000
    pad_idx: int | None = None
    tied_embeddings: bool = False
    num_layers: int = 32
    num_attn_heads: int = 32
    num_key_value_heads: int = 32
    ffn_inner_dim: int = 4096 * 4
    ffn_inner_dim_scale: float = 2 / 3
    ffn_inner_dim_multiplier: float = 1.0
    ffn_inner_dim_multiple_of: int = 256
    rope_theta: float = 10_000.0
    use_scaled_rope: bool = False
    rope_scale: LLaMARoPEScaleConfig = field(default_factory=LLaMARoPEScaleConfig)
    dropout_p: float = 0.0
    init_std: float | None = None
    init_std_scale: Literal["none", "layer", "stack"] = "layer"
    shard_embed_dim: bool = True


arch = ConfigRegistrar(LLaMAConfig)


@arch("7b")
def llama_7b() -> LLaMAConfig:
    return LLaMAConfig()


@arch("13b")
def llama_13b() -> LLaMAConfig:
    c = llama_7b()
    c.model_dim = 5120
    c.num_attn_heads = c.num_key_value_heads = 40
    c.num_layers = 40
    c.ffn_inner_dim = 5120 * 4
    return c


@arch("33b")
def llama_33b() -> LLaMAConfig:
    c = llama_7b()
    c.model_dim = 6656
    c.num_layers = 60
    c.num_attn_heads = c.num_key_value_heads = 52
    c.ffn_inner_dim = 6656 * 4
    return c


@arch("65b")
def llama_65b() -> LLaMAConfig:
    c = llama_7b()
    c.model_dim = 8192
    c.num_layers = 80
    c.num_attn_heads = c.num_key_value_heads = 64
    c.ffn_inner_dim = 8192 * 4
    return c


@arch("llama2_7b")
def llama2_7b() -> LLaMAConfig:
    c = llama_7b()
    c.max_seq_len = 4096
    return c


@arch("llama2_13b")
def llama2_13b() -> LLaMAConfig:
    c = llama_13b()
    c.max_seq_len = 4096
    return c


@arch("llama2_70b")
def llama2_70b() -> LLaMAConfig:
    c = llama_65b()
    c.max_seq_len = 4096
    c.num_key_value_heads = 8
    c.ffn_inner_dim = int(8192 * 4 * 1.3)
    c.ffn_inner_dim_multiple_of = 4096
    return c


@arch("llama3_8b")
def llama3_8b() -> LLaMAConfig:
    c = llama2_7b()
    c.max_seq_len = 8192
    c.vocab_size = 128_256
    c.pad_idx = 128_004
    c.num_key_value_heads = 8
    c.ffn_inner_dim = 4096 * 4
    c.ffn_inner_dim_multiplier = 1.3
    c.ffn_inner_dim_multiple_of = 1024
    c.rope_theta = 500_000.0
    c.shard_embed_dim = False
    return c


@arch("llama3_70b")
def llama3_70b() -> LLaMAConfig:
    c = llama2_70b()
    c.max_seq_len = 8192
    c.vocab_size = 128_256
    c.pad_idx = 128_004
    c.rope_theta = 500_000.0
    c.shard_embed_dim = False
    return c


@arch("llama3_1_8b")
def llama3_1_8b() -> LLaMAConfig:
    c = llama3_8b()
    c.max_seq_len = 131_072
    c.use_scaled_rope = True
    return c


@arch("llama3_1_70b")
def llama3_1_70b() -> LLaMAConfig:
    c = llama3_70b()
    c.max_seq_len = 131_072
    c.use_scaled_rope = True
    return c


@arch("llama3_2_3b")
def llama3_2_3b() -> LLaMAConfig:
    c = llama3_1_8b()
    c.model_dim = 3072
    c.ffn_inner_dim = int(3072 * 4 * 1.0)
    c.ffn_inner_dim_multiplier = 1.0
    c.ffn_inner_dim_multiple_of = 256
    c.num_attn_heads = 24
    c.num_key_value_heads = 8
    c.num_layers = 28
    c.rope_scale = LLaMARoPEScaleConfig(factor=32.0)
    c.tied_embeddings = True
    return c


@arch("llama3_2_1b")
def llama3_2_1b() -> LLaMAConfig:
    c = llama3_1_8b()
    c.model_dim = 2048
    c.ffn_inner_dim = int(2048 * 4 * 1.5)
    c.ffn_inner_dim_multiplier = 1.0
    c.ffn_inner_dim_multiple_of = 256
    c.num_attn_heads = 32
    c.num_key_value_heads = 8
    c.num_layers = 16
    c.rope_scale = LLaMARoPEScaleConfig(factor=32.0)
    c.tied_embeddings = True
    return c


@arch("tiny")
def llama_tiny() -> LLaMAConfig:
    """4-layer plumbing model used by the CPU/gloo end-to-end tests."""
    return LLaMAConfig(model_dim=256, max_seq_len=1024, vocab_size=8192, num_layers=4, num_attn_heads=4,
                       num_key_value_heads=2, ffn_inner_dim=688, ffn_inner_dim_scale=1.0,
                       ffn_inner_dim_multiple_of=1, rope_theta=10_000.0, shard_embed_dim=False)


def get_llama_config(name: str) -> LLaMAConfig:
    return get_config_registry(LLaMAConfig).get(name)
