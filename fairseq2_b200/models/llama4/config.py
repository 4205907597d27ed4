"""LLaMA-4 configuration (cf. fairseq2 ``models/llama4/config.py:23-106``)."""
from __future__ import annotations

from dataclasses import dataclass, field

from fairseq2_b200.models.llama.config import LLaMAConfig
from fairseq2_b200.runtime.config_registry import ConfigRegistrar

LLAMA4_FAMILY = "llama4"


@dataclass(kw_only=True)
class Llama4ExpertsConfig:
    num_experts: int = 16
    use_shared_expert: bool = True
    capacity_factor: float = 1.0
    auto_scale: bool = True
    """Shrink the expert width so that the activated parameters match an equivalent dense layer."""
    top_k: int = 1
    interleave_moe_layer_step: int = 1
    """Every n-th layer is a mixture of experts; 1 means every layer."""


@dataclass(kw_only=True)
class Llama4Config(LLaMAConfig):
    experts: Llama4ExpertsConfig = field(default_factory=Llama4ExpertsConfig)
    attention_chunk_size: int = 8192
    use_qk_norm: bool = False
    nope_layer_interval: int | None = None
    """Every n-th layer has no positional encoding and attends globally."""


arch = ConfigRegistrar(Llama4Config)


@arch("llama4_scout_17b_16e")
def llama4_scout_17b_16e() -> Llama4Config:
    c = Llama4Config(model_dim=5120, num_layers=48, num_attn_heads=40, num_key_value_heads=8, vocab_size=202_048,
                     pad_idx=200_018, ffn_inner_dim=5120 * 4, ffn_inner_dim_multiplier=1.2,
                     ffn_inner_dim_multiple_of=2048, use_qk_norm=True, rope_theta=500_000.0, use_scaled_rope=True,
                     nope_layer_interval=4, shard_embed_dim=False)
    c.rope_scale.factor = 16.0
    c.rope_scale.frequency_factors = (1.0, 1.0)
    return c


@arch("llama4_maverick_17b_128e")
def llama4_maverick_17b_128e() -> Llama4Config:
    c = llama4_scout_17b_16e()
    c.experts.num_experts = 128
    c.experts.interleave_moe_layer_step = 2
    c.use_qk_norm = False
    c.use_scaled_rope = False
    return c


@arch("tiny")
def llama4_tiny() -> Llama4Config:
    return Llama4Config(model_dim=128, max_seq_len=256, vocab_size=512, num_layers=4, num_attn_heads=4,
                        num_key_value_heads=2, ffn_inner_dim=512, ffn_inner_dim_multiple_of=32, use_qk_norm=True,
                        attention_chunk_size=32, nope_layer_interval=4, shard_embed_dim=False,
                        experts=Llama4ExpertsConfig(num_experts=4, top_k=1, interleave_moe_layer_step=2))
