"""Configuration of the mixture-of-experts decoder-only language model family: a LLaMA-style decoder (RMSNorm,
RoPE, grouped-query attention with an explicit head dimension) whose feed-forward layers are top-k routed SwiGLU
experts with softmax gates and a load-balancing auxiliary loss. The experts can be expert-parallel: rank ``r`` of
the expert-parallel gang owns experts ``[r * E / W, (r + 1) * E / W)``.

The reference has no expert parallelism and no auxiliary loss (its only MoE is LLaMA 4's sigmoid router with every
expert seeing every token, ``models/llama4/moe.py:109-157``); this family is the new capability that the
expert-parallel kernels of this framework serve."""
from __future__ import annotations

from dataclasses import dataclass

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

MOE_LM_FAMILY = "moe_lm"


@dataclass(kw_only=True)
class MoELMConfig:
    model_dim: int = 2048
    max_seq_len: int = 4096
    vocab_size: int = 151_936
    pad_idx: int | None = None
    num_layers: int = 48
    num_attn_heads: int = 32
    num_key_value_heads: int = 4
    head_dim: int = 128
    num_experts: int = 128
    expert_inner_dim: int = 768
    top_k: int = 8
    aux_loss_coef: float = 1e-3
    router_init_std: float = 0.02
    rope_theta: float = 1_000_000.0
    dropout_p: float = 0.0
    init_std: float | None = 0.02
    #: rows an expert-parallel inbox can hold, as a multiple of the mean load ``tokens * top_k`` per rank
    ep_capacity_factor: float = 2.0
    #: expert parallelism over the data-parallel gang: every rank builds ``num_experts / size`` experts and the
    #: tokens travel to them through the peer-memory dispatch / combine kernels (CUDA, 2 to 8 ranks of one node);
    #: ``False`` replicates the experts like any other parameter
    expert_parallel: bool = False
    #: most tokens one rank routes per forward pass when ``expert_parallel`` (sizes the dispatch buffers)
    ep_max_tokens: int = 16_384


arch = ConfigRegistrar(MoELMConfig)


@arch("qwen3_moe_30b_a3b")
def qwen3_moe_30b_a3b() -> MoELMConfig:
    """48 layers, model dim 2048, 32 query / 4 key-value heads of 128, 128 experts of inner dim 768, top-8."""
    return MoELMConfig()


@arch("tiny")
def tiny() -> MoELMConfig:
    return MoELMConfig(model_dim=128, max_seq_len=512, vocab_size=512, num_layers=2, num_attn_heads=4,
                       num_key_value_heads=2, head_dim=32, num_experts=8, expert_inner_dim=64, top_k=2)
