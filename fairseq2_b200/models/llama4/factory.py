"""Builds LLaMA-4 models (cf. fairseq2 ``models/llama4/factory.py:37-159``): the LLaMA decoder with
chunked local attention on RoPE layers, periodic global no-position layers, weight-free q/k RMSNorm and
mixture-of-experts feed-forward layers."""
from __future__ import annotations

from fairseq2_b200.gang import Gangs
from fairseq2_b200.models.llama.factory import LLaMAFactory, init_truncated_normal
from fairseq2_b200.models.llama4.config import Llama4Config
from fairseq2_b200.models.transformer.attention_bias import AttentionBias, CausalAttentionBias, ChunkedAttentionBias
from fairseq2_b200.models.transformer.experts import MoE
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention, StandardMultiheadAttention
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.transformer_lm import TransformerLM
from fairseq2_b200.nn.normalization import RMSNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder


def create_llama4_model(config: Llama4Config, gangs: Gangs | None = None) -> TransformerLM:
    return Llama4Factory(config, gangs).create_model()


class Llama4Factory(LLaMAFactory):
    _config: Llama4Config

    def _is_nope_layer(self, layer_idx: int) -> bool:
        n = self._config.nope_layer_interval
        return n is not None and (layer_idx + 1) % n == 0

    def create_self_attention(self, layer_idx: int, pos_encoder: PositionEncoder) -> MultiheadAttention:
        c = self._config
        nope = self._is_nope_layer(layer_idx)
        bias: AttentionBias
        if not nope and c.attention_chunk_size:
            bias = ChunkedAttentionBias(attn_chunk_size=c.attention_chunk_size)
        else:
            bias = CausalAttentionBias()
        hd = c.model_dim // c.num_attn_heads
        qk = (lambda: RMSNorm(hd, bias=False, elementwise_affine=False)) if (c.use_qk_norm and not nope) else (lambda: None)
        init = self._proj_init(layer_idx)
        return StandardMultiheadAttention(c.model_dim, c.num_attn_heads, create_default_sdpa(bias),
                                          num_key_value_heads=c.num_key_value_heads, qkv_proj_init_fn=init,
                                          q_norm=qk(), k_norm=qk(), pos_encoder=None if nope else pos_encoder,
                                          output_proj_init_fn=init, bias=False, gangs=self._gangs)

    def create_ffn(self, layer_idx: int) -> FeedForwardNetwork:
        c = self._config
        if (layer_idx + 1) % c.experts.interleave_moe_layer_step != 0:
            return super().create_ffn(layer_idx)
        e = c.experts
        return MoE(c.model_dim, int(c.ffn_inner_dim * c.ffn_inner_dim_multiplier), e.use_shared_expert,
                   e.num_experts, e.capacity_factor, e.top_k, inner_dim_scale=c.ffn_inner_dim_scale,
                   inner_dim_to_multiple=c.ffn_inner_dim_multiple_of, auto_scale=e.auto_scale, tp_gang=self._gangs.tp)
