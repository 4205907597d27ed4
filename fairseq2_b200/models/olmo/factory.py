"""Builds OLMo-2/3 models (cf. fairseq2 ``models/olmo/factory.py:56-420``,
``olmo/decoder_layer.py``, ``olmo/attention.py``, ``olmo/yarn_rope.py``).

Differences from LLaMA: the layer norm is applied to each sub-layer's OUTPUT
before the residual add; q/k RMSNorms span all heads; OLMo-3 interleaves
sliding-window and global layers and extends the context with YaRN-scaled RoPE.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from fairseq2_b200.gang import Gangs, get_current_gangs
from fairseq2_b200.models.olmo.config import OLMOConfig, YaRNScaleConfig
from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache, CausalAttentionBias
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork, GLUFeedForwardNetwork
from fairseq2_b200.models.transformer.frontend import TransformerEmbeddingFrontend
from fairseq2_b200.models.transformer.multihead_attention import (LocalAttentionState, MultiheadAttention,
                                                                  StandardMultiheadAttention)
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.transformer_lm import StandardTransformerLMDecoder, TransformerLM, TransformerLMDecoderLayer
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.embedding import StandardEmbedding
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm, RMSNorm
from fairseq2_b200.nn.position_encoder import RotaryEncoder
from fairseq2_b200.nn.projection import Linear, Projection, TiedProjection
from fairseq2_b200.nn.residual import AdditiveResidualConnect


class OLMOTransformerLMDecoderLayer(TransformerLMDecoderLayer):
    """``x + norm(attn(x))`` then ``x + norm(ffn(x))``."""

    def __init__(self, self_attn: MultiheadAttention, self_attn_layer_norm: LayerNorm, ffn: FeedForwardNetwork,
                 ffn_layer_norm: LayerNorm, *, dropout_p: float = 0.0) -> None:
        super().__init__()
        self.self_attn, self.self_attn_layer_norm = self_attn, self_attn_layer_norm
        self.ffn, self.ffn_layer_norm = ffn, ffn_layer_norm
        self.self_attn_residual, self.ffn_residual = AdditiveResidualConnect(), AdditiveResidualConnect()
        self.dropout = torch.nn.Dropout(dropout_p) if dropout_p > 0.0 else None

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, bias_cache: AttentionBiasCache, *,  # type: ignore[override]
                state_bag: IncrementalStateBag | None = None) -> Tensor:
        residual = seqs
        seqs = self.self_attn(seqs, seqs_layout, seqs, seqs_layout, seqs, bias_cache, state_bag=state_bag)
        if self.dropout is not None:
            seqs = self.dropout(seqs)
        seqs = self.self_attn_residual(self.self_attn_layer_norm(seqs), residual)
        residual = seqs
        seqs = self.ffn(seqs)
        if self.dropout is not None:
            seqs = self.dropout(seqs)
        return self.ffn_residual(self.ffn_layer_norm(seqs), residual)


def yarn_attention_scaling(y: YaRNScaleConfig) -> float:
    def mscale(scale: float, m: float) -> float:
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    if y.mscale and y.mscale_all_dim:
        return mscale(y.scale_factor, y.mscale) / mscale(y.scale_factor, y.mscale_all_dim)
    return mscale(y.scale_factor, y.mscale or 1.0)


def yarn_inv_freqs(dim: int, theta: float, y: YaRNScaleConfig, device: torch.device) -> Tensor:
    """High-frequency pairs keep their wavelength, low-frequency pairs are stretched by ``scale_factor``,
    with a linear ramp between the ``beta_fast`` and ``beta_slow`` rotation counts."""
    def correction_dim(num_rot: float) -> float:
        return dim * math.log(y.original_max_seq_len / (num_rot * 2 * math.pi)) / (2 * math.log(theta))

    low, high = correction_dim(y.beta_fast), correction_dim(y.beta_slow)
    if y.truncate:
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, dim - 1)
    if low == high:
        high += 0.001
    pos = theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim)
    ramp = 1 - ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
    return (1.0 / (y.scale_factor * pos)) * (1 - ramp) + (1.0 / pos) * ramp


class YaRNRotaryEncoder(RotaryEncoder):
    """RoPE whose inverse frequencies follow YaRN; the attention-temperature correction is folded
    into the (cos, sin) table so that q and k are both scaled by it."""

    def __init__(self, encoding_dim: int, max_seq_len: int, *, theta: float, scale: YaRNScaleConfig,
                 device: torch.device | None = None) -> None:
        self.yarn = scale
        self.attention_scaling = yarn_attention_scaling(scale)
        super().__init__(encoding_dim, max_seq_len, theta=theta,
                         freqs_init_fn=lambda pe: yarn_inv_freqs(pe.encoding_dim, pe.theta, scale, pe.freqs.device),
                         device=device)

    def reset_non_persistent_buffers(self) -> None:
        super().reset_non_persistent_buffers()
        if self.freqs.device.type != "meta":
            self.freqs.mul_(self.attention_scaling)


def create_olmo_model(config: OLMOConfig, gangs: Gangs | None = None) -> TransformerLM:
    c = config
    gangs = gangs if gangs is not None else get_current_gangs()
    hd = c.model_dim // c.num_attn_heads
    eps = c.rms_norm_eps

    def trunc(w: Tensor, b: Tensor | None, std: float) -> None:
        torch.nn.init.trunc_normal_(w, mean=0.0, std=std, a=-3 * std, b=3 * std)
        if b is not None:
            torch.nn.init.zeros_(b)

    embed = StandardEmbedding(c.vocab_size, c.model_dim, c.pad_idx,
                              init_fn=lambda e: trunc(e.weight, None, c.init_std or c.model_dim ** -0.5))
    frontend = TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=None, no_scale=True,
                                            dropout_p=c.dropout_p)
    if c.yarn_scale_config is not None:
        pe: RotaryEncoder = YaRNRotaryEncoder(hd, c.max_seq_len, theta=c.rope_theta, scale=c.yarn_scale_config)
    else:
        pe = RotaryEncoder(hd, c.max_seq_len, theta=c.rope_theta)
    types = c.resolved_layer_types()
    layers = []
    for i in range(c.num_layers):
        if c.init_std_scale == "none":
            s = 1.0
        elif c.init_std_scale == "layer":
            s = (2 * (i + 1)) ** 0.5
        else:
            s = (2 * (c.num_layers + 1)) ** 0.5

        def init(p: Linear, s: float = s) -> None:
            trunc(p.weight, p.bias, (c.init_std or p.weight.shape[1] ** -0.5) / s)

        sliding = types[i] == "sliding_attention"
        window = c.sliding_window if sliding else None
        factory = None
        if window is not None:
            def factory(k, v, max_seq_len, capacity_increment, w=window):  # type: ignore[no-untyped-def,misc]
                return LocalAttentionState(k, v, max_seq_len, w, capacity_increment)

        attn = StandardMultiheadAttention(
            c.model_dim, c.num_attn_heads, create_default_sdpa(CausalAttentionBias(attn_window_len=window)),
            num_key_value_heads=c.num_key_value_heads, qkv_proj_init_fn=init,
            q_norm=RMSNorm(c.num_attn_heads * hd, bias=False, eps=eps),
            k_norm=RMSNorm(c.num_key_value_heads * hd, bias=False, eps=eps), qk_norm_over_heads=True,
            pos_encoder=pe, output_proj_init_fn=init, bias=False, state_factory=factory, gangs=gangs)
        ffn = GLUFeedForwardNetwork(c.model_dim, c.ffn_inner_dim, bias=False, inner_dim_scale=1.0, proj_init_fn=init,
                                    gangs=gangs)
        layers.append(OLMOTransformerLMDecoderLayer(attn, RMSNorm(c.model_dim, bias=False, eps=eps), ffn,
                                                    RMSNorm(c.model_dim, bias=False, eps=eps), dropout_p=c.dropout_p))
    decoder = StandardTransformerLMDecoder(layers, RMSNorm(c.model_dim, bias=False, eps=eps))
    final: Projection
    if c.tied_embeddings:
        final = TiedProjection(embed.weight, bias=None)
    else:
        final = Linear(c.model_dim, c.vocab_size, bias=False,
                       init_fn=lambda p: trunc(p.weight, None, c.init_std or c.model_dim ** -0.5))
    return TransformerLM(c.model_dim, frontend, decoder, final, c.pad_idx, c.max_seq_len)
