"""Builds LLaMA models (cf. fairseq2 ``models/llama/factory.py:56-335``).

Tensor-parallel sharding is decided inside the factory from the current gangs:
q/k/v/gate/up are column-sharded, o/down row-sharded, the embedding
vocabulary-sharded (or dimension-sharded for LLaMA-1/2) and the output
projection column-sharded with gathered output.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.gang import Gangs, get_current_gangs
from fairseq2_b200.models.llama.config import LLaMAConfig, LLaMARoPEScaleConfig
from fairseq2_b200.models.transformer.attention_bias import CausalAttentionBias
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork, GLUFeedForwardNetwork
from fairseq2_b200.models.transformer.frontend import TransformerEmbeddingFrontend, TransformerFrontend
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention, StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.transformer_lm import (StandardTransformerLMDecoder, StandardTransformerLMDecoderLayer,
                                                 TransformerLM, TransformerLMDecoder, TransformerLMDecoderLayer)
from fairseq2_b200.nn.embedding import Embedding, ShardedEmbedding, StandardEmbedding, VocabShardedEmbedding
from fairseq2_b200.nn.normalization import LayerNorm, RMSNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder, RotaryEncoder
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, Projection, TiedProjection


def create_llama_model(config: LLaMAConfig, gangs: Gangs | None = None) -> TransformerLM:
    return LLaMAFactory(config, gangs).create_model()


def init_truncated_normal(weight: Tensor, bias: Tensor | None, *, std: float = 1.0) -> None:
    torch.nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
    if bias is not None:
        torch.nn.init.zeros_(bias)


class LLaMAFactory:
    def __init__(self, config: LLaMAConfig, gangs: Gangs | None = None) -> None:
        self._config = config
        self._gangs = gangs if gangs is not None else get_current_gangs()
        from fairseq2_b200.parallel.tp import sequence_parallel_enabled

        # training-time layout of tensor parallelism: the residual stream is sharded over the tokens
        self._sequence_parallel = self._gangs.tp.size > 1 and sequence_parallel_enabled()

    def create_model(self) -> TransformerLM:
        c = self._config
        embed = self.create_embedding()
        model = TransformerLM(c.model_dim, self.create_decoder_frontend(embed), self.create_decoder(),
                              self.create_final_projection(embed), c.pad_idx, c.max_seq_len)
        model.tp_sequence_parallel = self._sequence_parallel
        return model

    def create_embedding(self) -> Embedding:
        c = self._config
        init_std = c.init_std

        def init_embed(e: StandardEmbedding) -> None:
            init_truncated_normal(e.weight, None, std=init_std or e.weight.shape[1] ** -0.5)

        tp = self._gangs.tp
        if tp.size == 1:
            return StandardEmbedding(c.vocab_size, c.model_dim, c.pad_idx, init_fn=init_embed)
        if c.shard_embed_dim:
            if self._sequence_parallel:
                raise NotSupportedError("Sequence-parallel tensor parallelism needs a vocabulary-sharded embedding "
                                        "(`shard_embed_dim=False`).")
            return ShardedEmbedding(tp, c.vocab_size, c.model_dim, c.pad_idx, init_fn=init_embed)
        return VocabShardedEmbedding(tp, c.vocab_size, c.model_dim, c.pad_idx,
                                     sequence_parallel=self._sequence_parallel, init_fn=init_embed)

    def create_decoder_frontend(self, embed: Embedding) -> TransformerFrontend:
        c = self._config
        return TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=None, no_scale=True,
                                            dropout_p=c.dropout_p)

    def create_decoder(self) -> TransformerLMDecoder:
        c = self._config
        pe = self.create_position_encoder()
        layers = [self.create_decoder_layer(i, pe) for i in range(c.num_layers)]
        return StandardTransformerLMDecoder(layers, self.create_layer_norm())

    def create_position_encoder(self) -> PositionEncoder:
        c = self._config
        fn = None
        if c.use_scaled_rope:
            scale = c.rope_scale

            def fn(pe: RotaryEncoder) -> Tensor:  # type: ignore[misc]
                return init_llama_rope_freqs(pe, scale)

        return RotaryEncoder(c.model_dim // c.num_attn_heads, c.max_seq_len, theta=c.rope_theta, freqs_init_fn=fn)

    def create_decoder_layer(self, layer_idx: int, pos_encoder: PositionEncoder) -> TransformerLMDecoderLayer:
        c = self._config
        return StandardTransformerLMDecoderLayer(
            self.create_self_attention(layer_idx, pos_encoder), self.create_layer_norm(),
            self.create_ffn(layer_idx), self.create_layer_norm(), norm_order=TransformerNormOrder.PRE,
            dropout_p=c.dropout_p)

    def _proj_init(self, layer_idx: int):  # type: ignore[no-untyped-def]
        init_std = self._config.init_std
        scale = self.get_std_scale_factor(layer_idx)

        def init(p: Linear) -> None:
            init_truncated_normal(p.weight, p.bias, std=(init_std or p.weight.shape[1] ** -0.5) / scale)

        return init

    def create_self_attention(self, layer_idx: int, pos_encoder: PositionEncoder) -> MultiheadAttention:
        c = self._config
        init = self._proj_init(layer_idx)
        return StandardMultiheadAttention(c.model_dim, c.num_attn_heads, create_default_sdpa(CausalAttentionBias()),
                                          num_key_value_heads=c.num_key_value_heads, qkv_proj_init_fn=init,
                                          pos_encoder=pos_encoder, output_proj_init_fn=init, bias=False,
                                          gangs=self._gangs)

    def create_ffn(self, layer_idx: int) -> FeedForwardNetwork:
        c = self._config
        return GLUFeedForwardNetwork(c.model_dim, int(c.ffn_inner_dim * c.ffn_inner_dim_multiplier), bias=False,
                                     inner_dim_scale=c.ffn_inner_dim_scale,
                                     inner_dim_to_multiple=c.ffn_inner_dim_multiple_of,
                                     proj_init_fn=self._proj_init(layer_idx), gangs=self._gangs)

    def create_final_projection(self, embed: Embedding) -> Projection:
        c = self._config
        tp = self._gangs.tp
        if c.tied_embeddings:
            if tp.size > 1:
                raise NotSupportedError("Tied embeddings are not supported when tensor parallelism is enabled.")
            if not isinstance(embed, StandardEmbedding):
                raise TypeError("`embed` must be a `StandardEmbedding` when `tied_embeddings` is set.")
            return TiedProjection(embed.weight, bias=None)
        init_std = c.init_std

        def init(p: Linear) -> None:
            init_truncated_normal(p.weight, p.bias, std=init_std or p.weight.shape[1] ** -0.5)

        if tp.size == 1:
            return Linear(c.model_dim, c.vocab_size, bias=False, init_fn=init)
        return ColumnShardedLinear(tp, c.model_dim, c.vocab_size, bias=False, gather_output=True,
                                   sequence_parallel=self._sequence_parallel, init_fn=init)

    def create_layer_norm(self) -> LayerNorm:
        return RMSNorm(self._config.model_dim, bias=False)

    def get_std_scale_factor(self, layer_idx: int) -> float:
        c = self._config
        if c.init_std_scale == "none":
            return 1.0
        if c.init_std_scale == "layer":
            n = layer_idx
        elif c.init_std_scale == "stack":
            n = c.num_layers
        else:
            raise ValueError(
                f"`config.init_std_scale` must be 'none', 'layer', or 'stack', but is '{c.init_std_scale}' instead.")
        return (2 * (n + 1)) ** 0.5


def init_llama_rope_freqs(pos_encoder: RotaryEncoder, rope_scale: LLaMARoPEScaleConfig) -> Tensor:
    """Inverse frequencies with LLaMA-3.1 smoothing: wavelengths shorter than
    ``ctx/high`` are kept, longer than ``ctx/low`` are divided by ``factor``,
    the band in between is interpolated."""
    dev = pos_encoder.freqs.device
    idx = torch.arange(0, pos_encoder.encoding_dim, 2, device=dev, dtype=torch.float32)
    freqs = 1.0 / (pos_encoder.theta ** (idx / pos_encoder.encoding_dim))
    if dev.type == "meta":
        return freqs
    ctx = rope_scale.original_context_length
    lo, hi = rope_scale.frequency_factors
    wavelen = 2 * math.pi / freqs
    smooth = ((ctx / wavelen) - lo) / (hi - lo)
    mid = (1 - smooth) * freqs / rope_scale.factor + smooth * freqs
    out = torch.where(wavelen < ctx / hi, freqs, torch.where(wavelen > ctx / lo, freqs / rope_scale.factor, mid))
    return out
