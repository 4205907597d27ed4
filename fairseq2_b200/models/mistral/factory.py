"""Builds Mistral models (cf. fairseq2 ``models/mistral/factory.py:43-178``): LLaMA-style pre-norm
decoder with grouped-query sliding-window attention and a rolling KV cache for generation."""
from __future__ import annotations

import torch

from fairseq2_b200.gang import Gangs, get_current_gangs
from fairseq2_b200.models.mistral.config import MistralConfig
from fairseq2_b200.models.transformer.attention_bias import CausalAttentionBias
from fairseq2_b200.models.transformer.ffn import GLUFeedForwardNetwork
from fairseq2_b200.models.transformer.frontend import TransformerEmbeddingFrontend
from fairseq2_b200.models.transformer.multihead_attention import LocalAttentionState, StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.transformer_lm import (StandardTransformerLMDecoder, StandardTransformerLMDecoderLayer,
                                                 TransformerLM)
from fairseq2_b200.nn.embedding import StandardEmbedding
from fairseq2_b200.nn.normalization import RMSNorm
from fairseq2_b200.nn.position_encoder import RotaryEncoder
from fairseq2_b200.nn.projection import Linear


def _init_final_projection(p: Linear) -> None:
    torch.nn.init.normal_(p.weight, std=p.weight.shape[1] ** -0.5)
    if p.bias is not None:
        torch.nn.init.zeros_(p.bias)


def create_mistral_model(config: MistralConfig, gangs: Gangs | None = None) -> TransformerLM:
    c = config
    gangs = gangs if gangs is not None else get_current_gangs()
    embed = StandardEmbedding(c.vocab_size, c.model_dim, c.pad_idx)
    frontend = TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=None, no_scale=True,
                                            dropout_p=c.dropout_p)
    pe = RotaryEncoder(c.model_dim // c.num_attn_heads, c.max_seq_len, theta=c.rope_theta)
    window = c.attn_window_len

    def state_factory(k, v, max_seq_len, capacity_increment):  # type: ignore[no-untyped-def]
        return LocalAttentionState(k, v, max_seq_len, window, capacity_increment)

    layers = []
    for _ in range(c.num_layers):
        attn = StandardMultiheadAttention(
            c.model_dim, c.num_attn_heads, create_default_sdpa(CausalAttentionBias(attn_window_len=window)),
            num_key_value_heads=c.num_key_value_heads, pos_encoder=pe, bias=False, state_factory=state_factory,
            gangs=gangs)
        ffn = GLUFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=False, inner_dim_scale=1.0, gangs=gangs)
        layers.append(StandardTransformerLMDecoderLayer(
            attn, RMSNorm(c.model_dim, bias=False), ffn, RMSNorm(c.model_dim, bias=False),
            norm_order=TransformerNormOrder.PRE, dropout_p=c.dropout_p))
    decoder = StandardTransformerLMDecoder(layers, RMSNorm(c.model_dim, bias=False))
    final = Linear(c.model_dim, c.vocab_size, bias=False, init_fn=_init_final_projection)
    return TransformerLM(c.model_dim, frontend, decoder, final, c.pad_idx, c.max_seq_len)
