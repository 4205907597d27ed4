"""Builds Qwen models (cf. fairseq2 ``models/qwen/factory.py:48-245``): pre-norm decoder with
grouped-query attention, q/k/v biases (2.5) or per-head q/k RMSNorm (3), SwiGLU FFN, RMSNorm eps 1e-6."""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.gang import Gangs, get_current_gangs
from fairseq2_b200.models.qwen.config import QwenConfig
from fairseq2_b200.models.transformer.attention_bias import CausalAttentionBias
from fairseq2_b200.models.transformer.ffn import GLUFeedForwardNetwork
from fairseq2_b200.models.transformer.frontend import TransformerEmbeddingFrontend
from fairseq2_b200.models.transformer.multihead_attention import StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.transformer_lm import (StandardTransformerLMDecoder, StandardTransformerLMDecoderLayer,
                                                 TransformerLM)
from fairseq2_b200.nn.embedding import StandardEmbedding, VocabShardedEmbedding
from fairseq2_b200.nn.normalization import RMSNorm
from fairseq2_b200.nn.position_encoder import RotaryEncoder
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, Projection, TiedProjection

_EPS = 1e-6


def _trunc(weight: Tensor, bias: Tensor | None, std: float) -> None:
    torch.nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
    if bias is not None:
        torch.nn.init.zeros_(bias)


def create_qwen_model(config: QwenConfig, gangs: Gangs | None = None) -> TransformerLM:
    c = config
    gangs = gangs if gangs is not None else get_current_gangs()
    tp = gangs.tp
    hd = c.head_dim if c.head_dim is not None else c.model_dim // c.num_attn_heads

    def init_embed(e: StandardEmbedding) -> None:
        _trunc(e.weight, None, c.model_dim ** -0.5)

    if tp.size == 1:
        embed = StandardEmbedding(c.vocab_size, c.model_dim, init_fn=init_embed)
    else:
        embed = VocabShardedEmbedding(tp, c.vocab_size, c.model_dim, init_fn=init_embed)
    frontend = TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=None, no_scale=True,
                                            dropout_p=c.dropout_p)
    pe = RotaryEncoder(hd, c.max_seq_len, theta=c.rope_theta)
    layers = []
    for i in range(c.num_layers):
        std_scale = (2 * (i + 1)) ** 0.5

        def init(p: Linear, s: float = std_scale) -> None:
            _trunc(p.weight, p.bias, p.weight.shape[1] ** -0.5 / s)

        attn = StandardMultiheadAttention(
            c.model_dim, c.num_attn_heads, create_default_sdpa(CausalAttentionBias()), head_dim=hd,
            num_key_value_heads=c.num_key_value_heads, qkv_proj_init_fn=init,
            q_norm=RMSNorm(hd, bias=False, eps=_EPS) if c.q_norm else None,
            k_norm=RMSNorm(hd, bias=False, eps=_EPS) if c.k_norm else None, pos_encoder=pe,
            output_proj_init_fn=init, bias=c.qkv_proj_bias, output_proj_bias=False, gangs=gangs)
        ffn = GLUFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=False, inner_dim_scale=1.0, proj_init_fn=init,
                                    gangs=gangs)
        layers.append(StandardTransformerLMDecoderLayer(
            attn, RMSNorm(c.model_dim, bias=False, eps=_EPS), ffn, RMSNorm(c.model_dim, bias=False, eps=_EPS),
            norm_order=TransformerNormOrder.PRE, dropout_p=c.dropout_p))
    decoder = StandardTransformerLMDecoder(layers, RMSNorm(c.model_dim, bias=False, eps=_EPS))
    final: Projection
    if c.tied_embeddings:
        if tp.size > 1:
            raise NotSupportedError("Tied embeddings are not supported when tensor parallelism is enabled.")
        final = TiedProjection(embed.weight, bias=None)
    elif tp.size == 1:
        final = Linear(c.model_dim, c.vocab_size, bias=False, init_fn=lambda p: _trunc(p.weight, None, c.model_dim ** -0.5))
    else:
        final = ColumnShardedLinear(tp, c.model_dim, c.vocab_size, bias=False, gather_output=True,
                                    init_fn=lambda p: _trunc(p.weight, None, c.model_dim ** -0.5))
    return TransformerLM(c.model_dim, frontend, decoder, final, None, c.max_seq_len)
