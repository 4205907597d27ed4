"""Gemma 3n audio tower: mel frames -> two strided 2-D convolutions with cumulative group norm -> conformer blocks
(macaron feed-forward, local attention with relative position bias and logit soft-cap, gated causal depthwise
convolution) -> 4x temporal reduction, and the embedder that maps tower outputs (or audio token ids) into the
text model's embedding space (cf. fairseq2 ``models/gemma3n/audio/{subsample,conformer,sdpa,tower,embedder}.py``).

Local attention is evaluated as one banded attention over the whole sequence: query ``i`` sees keys
``i - (context_left - 1) <= j <= i + context_right``, with bias ``q_i . P(i - j)`` where ``P(d)`` is a projected
sinusoidal embedding of the distance -- the same numbers as the chunked formulation without its unfold/pad copies.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Conv1d, Conv2d, Embedding, Module, ModuleList, Parameter

from fairseq2_b200.models.gemma3n.config import Gemma3nAudioConfig
from fairseq2_b200.nn.normalization import RMSNorm
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.typing import DataType, Device


def _norm(dim: int, eps: float, kw: dict) -> RMSNorm:  # type: ignore[type-arg]
    return RMSNorm(dim, bias=False, eps=eps, **kw)


class RelativePositionEmbedding(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        self.heads, self.channels = cfg.conf_num_attention_heads, cfg.hidden_size
        self.head_dim = self.channels // self.heads
        self.max_backward = max(0, cfg.conf_attention_context_left - 1)
        self.max_forward = cfg.conf_attention_context_right
        self.pos_proj = Linear(self.channels, self.heads * self.head_dim, bias=False, **kw)

    def distance_embeddings(self, dtype: torch.dtype, device: torch.device) -> Tensor:
        """``[F, heads, head_dim]`` for distances ``max_backward, ..., -max_forward`` (in that order)."""
        half = self.channels // 2
        inc = math.log(1.0e4) / max(half - 1, 1)
        inv = torch.exp(torch.arange(half, device=device, dtype=torch.float32) * -inc)
        d = torch.arange(self.max_backward, -self.max_forward - 1, -1, device=device, dtype=torch.float32)
        ang = d.unsqueeze(-1) * inv
        timing = torch.cat([torch.sin(ang), torch.cos(ang)], dim=-1).to(dtype)
        return self.pos_proj(timing).view(-1, self.heads, self.head_dim)


class LocalAttention(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        self.heads, self.hidden = cfg.conf_num_attention_heads, cfg.hidden_size
        self.head_dim = self.hidden // self.heads
        self.past = max(0, cfg.conf_attention_context_left - 1)
        self.future = cfg.conf_attention_context_right
        self.cap = cfg.conf_attention_logit_cap
        self.relative_position_embedding = RelativePositionEmbedding(cfg, kw)
        self.per_dim_scale = Parameter(torch.zeros(self.head_dim, **kw))
        self.q_proj = Linear(self.hidden, self.hidden, bias=False, **kw)
        self.k_proj = Linear(self.hidden, self.hidden, bias=False, **kw)
        self.v_proj = Linear(self.hidden, self.hidden, bias=False, **kw)
        self.q_scale = self.head_dim ** -0.5 / math.log(2.0)              # 1 / softplus(0) = 1 / ln 2

    def forward(self, x: Tensor, invalid: Tensor) -> Tensor:
        """``x``: ``[B, T, hidden]``, ``invalid``: ``[B, T]`` (True = padding) -> ``[B, T, heads, head_dim]``."""
        B, T, _ = x.shape
        shape = (B, T, self.heads, self.head_dim)
        q = self.q_proj(x).view(shape) * self.q_scale * F.softplus(self.per_dim_scale)
        k, v = self.k_proj(x).view(shape), self.v_proj(x).view(shape)
        logits = torch.einsum("bthd,bshd->bhts", q, k)
        emb = self.relative_position_embedding.distance_embeddings(q.dtype, q.device)      # [F, h, d]
        by_distance = torch.einsum("bthd,fhd->bhtf", q, emb)                                # column f <-> distance past - f
        t = torch.arange(T, device=x.device)
        dist = t.unsqueeze(1) - t.unsqueeze(0)                                              # i - j
        in_band = (dist <= self.past) & (dist >= -self.future)
        col = (self.past - dist).clamp(0, emb.shape[0] - 1)
        logits = logits + by_distance.gather(-1, col.expand(B, self.heads, T, T))
        logits = torch.tanh(logits / self.cap) * self.cap
        allowed = in_band.view(1, 1, T, T) & ~invalid.view(B, 1, 1, T)
        logits = torch.where(allowed, logits, torch.finfo(logits.dtype).min)
        probs = torch.softmax(logits, dim=-1, dtype=torch.float32).to(v.dtype)
        return torch.einsum("bhts,bshd->bthd", probs, v)


class CumulativeGroupNorm(Module):
    """Normalisation whose mean and variance at frame ``t`` are taken over all features of frames ``0..t``."""

    def __init__(self, num_channels: int, feature_dims: tuple[int, ...], eps: float, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        self.num_channels, self.feature_dims, self.eps = num_channels, tuple(feature_dims), eps
        self.weight = Parameter(torch.ones(num_channels, **kw))

    def forward(self, x: Tensor) -> Tensor:
        """``x``: ``[B, T, *feature_dims, C]``."""
        xf = x.float()
        axes = tuple(range(2, x.dim()))
        per_frame = float(math.prod(x.shape[2:]))
        count = torch.arange(1, x.shape[1] + 1, device=x.device, dtype=torch.float32).view(1, -1, *([1] * (x.dim() - 2)))
        count = count * per_frame
        mean = torch.cumsum(xf.sum(dim=axes, keepdim=True), dim=1) / count
        var = torch.cumsum((xf - mean).pow(2).sum(dim=axes, keepdim=True), dim=1) / count
        return ((xf - mean) * torch.rsqrt(var + self.eps) * self.weight.float()).to(x.dtype)


class SSCPConvBlock(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, idx: int, input_freq_dim: int, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        kh, kw_ = cfg.sscp_conv_kernel_size[idx]
        sh, sw = cfg.sscp_conv_stride_size[idx]
        in_ch = 1 if idx == 0 else cfg.sscp_conv_channel_size[idx - 1]
        out_ch = cfg.sscp_conv_channel_size[idx]
        self.padding = (1, 1, 0, kh - 1)                      # (freq left, freq right, time top, time bottom)
        self.conv = Conv2d(in_ch, out_ch, (kh, kw_), stride=(sh, sw), bias=False, **kw)
        self.out_freq_dim = (input_freq_dim + 2 - kw_) // sw + 1
        self.norm = CumulativeGroupNorm(out_ch, (self.out_freq_dim,), cfg.sscp_conv_group_norm_eps, kw)

    def forward(self, x: Tensor) -> Tensor:
        """``[B, C_in, T, F]`` -> ``[B, C_out, T', F']``."""
        y = self.conv(F.pad(x, self.padding).to(self.conv.weight.dtype))
        y = self.norm(y.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)
        return F.relu(y)


class SubSampleConvProjection(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        self.conv_0 = SSCPConvBlock(cfg, 0, cfg.input_feat_size, kw)
        self.conv_1 = SSCPConvBlock(cfg, 1, self.conv_0.out_freq_dim, kw)
        self.input_proj_linear = Linear(cfg.sscp_conv_channel_size[-1] * self.conv_1.out_freq_dim, cfg.hidden_size,
                                        bias=False, **kw)

    def forward(self, mel: Tensor) -> Tensor:
        """``[B, T, mel_bins]`` -> ``[B, T / 4, hidden]``."""
        x = self.conv_1(self.conv_0(mel.unsqueeze(1)))
        b, c, t, f = x.shape
        return self.input_proj_linear(x.permute(0, 2, 3, 1).reshape(b, t, f * c))


class ConformerFeedForward(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        h = cfg.hidden_size
        self.clip, self.scale = cfg.gradient_clipping, cfg.conf_residual_weight
        self.pre_layer_norm, self.post_layer_norm = _norm(h, 1e-6, kw), _norm(h, 1e-6, kw)
        self.ffw_layer_1 = Linear(h, 4 * h, bias=False, **kw)
        self.ffw_layer_2 = Linear(4 * h, h, bias=False, **kw)

    def forward(self, x: Tensor) -> Tensor:
        y = self.pre_layer_norm(x.clamp(-self.clip, self.clip))
        y = self.ffw_layer_2(F.silu(self.ffw_layer_1(y))).clamp(-self.clip, self.clip)
        return x + self.post_layer_norm(y) * self.scale


class ConformerAttention(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        h = cfg.hidden_size
        self.clip = cfg.gradient_clipping
        self.pre_attn_norm, self.post_norm = _norm(h, 1e-6, kw), _norm(h, 1e-6, kw)
        self.attn = LocalAttention(cfg, kw)
        self.post = Linear(h, h, bias=False, **kw)

    def forward(self, x: Tensor, invalid: Tensor) -> Tensor:
        y = self.attn(self.pre_attn_norm(x.clamp(-self.clip, self.clip)), invalid)
        y = self.post(y.reshape(*y.shape[:2], -1)).clamp(-self.clip, self.clip)
        return x + self.post_norm(y)


class ConformerLightConv1d(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        h = cfg.hidden_size
        self.clip, self.causal_padding = cfg.gradient_clipping, cfg.conf_conv_kernel_size - 1
        self.pre_layer_norm, self.conv_norm = _norm(h, cfg.rms_norm_eps, kw), _norm(h, cfg.rms_norm_eps, kw)
        self.linear_start = Linear(h, 2 * h, bias=False, **kw)
        self.depthwise_conv1d = Conv1d(h, h, cfg.conf_conv_kernel_size, groups=h, bias=False, **kw)
        self.linear_end = Linear(h, h, bias=False, **kw)

    def forward(self, x: Tensor) -> Tensor:
        y = F.glu(self.linear_start(self.pre_layer_norm(x)), dim=-1)
        y = self.depthwise_conv1d(F.pad(y.transpose(1, 2), (self.causal_padding, 0))).transpose(1, 2)
        y = self.conv_norm(y.clamp(-self.clip, self.clip))
        return self.linear_end(F.silu(y)) + x


class ConformerBlock(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, kw: dict) -> None:  # type: ignore[type-arg]
        super().__init__()
        self.clip = cfg.gradient_clipping
        self.ffw_layer_start = ConformerFeedForward(cfg, kw)
        self.attention = ConformerAttention(cfg, kw)
        self.lconv1d = ConformerLightConv1d(cfg, kw)
        self.ffw_layer_end = ConformerFeedForward(cfg, kw)
        self.norm = _norm(cfg.hidden_size, 1e-6, kw)

    def forward(self, x: Tensor, invalid: Tensor) -> Tensor:
        x = self.attention(self.ffw_layer_start(x), invalid)
        x = self.lconv1d(x * (~invalid).unsqueeze(-1).to(x.dtype))
        return self.norm(self.ffw_layer_end(x).clamp(-self.clip, self.clip))


class Gemma3nAudioEncoder(Module):
    def __init__(self, cfg: Gemma3nAudioConfig, *, device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.cfg = cfg
        self.subsample_conv_projection = SubSampleConvProjection(cfg, kw)
        self.conformer = ModuleList([ConformerBlock(cfg, kw) for _ in range(cfg.conf_num_hidden_layers)])

    def forward(self, mel: Tensor, mel_invalid: Tensor) -> tuple[Tensor, Tensor]:
        """``mel``: ``[B, frames, mel_bins]``, ``mel_invalid``: ``[B, frames]`` (True = padding). Returns the audio
        encodings ``[B, frames / 16, hidden]`` (zero at padded positions) and their padding mask."""
        x = self.subsample_conv_projection(mel)
        stride = 1
        for s in self.cfg.sscp_conv_stride_size:
            stride *= s[0]
        idx = (torch.arange(x.shape[1], device=mel.device) * stride).clamp(max=mel_invalid.shape[1] - 1)
        invalid = mel_invalid[:, idx]
        for block in self.conformer:
            x = block(x, invalid)
        r = self.cfg.conf_reduction_factor
        if r > 1:
            x, invalid = x[:, ::r], invalid[:, ::r]
        return x.masked_fill(invalid.unsqueeze(-1), 0.0), invalid


class Gemma3nMultimodalEmbedder(Module):
    """Audio soft tokens (tower outputs) or audio hard tokens (ids in the audio vocabulary range) -> text embedding
    space: norm -> projection -> scale-free norm."""

    def __init__(self, cfg: Gemma3nAudioConfig, text_dim: int, *, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.vocab_offset, self.eps = cfg.vocab_offset, cfg.rms_norm_eps
        self.embedding = Embedding(cfg.vocab_size, cfg.hidden_size, **kw)
        self.hard_embedding_norm = _norm(cfg.hidden_size, cfg.rms_norm_eps, kw)
        self.soft_embedding_norm = _norm(cfg.hidden_size, cfg.rms_norm_eps, kw)
        self.embedding_projection = Linear(cfg.hidden_size, text_dim, bias=False, **kw)

    def forward(self, input_ids: Tensor | None = None, inputs_embeds: Tensor | None = None) -> Tensor:
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("Exactly one of `input_ids` and `inputs_embeds` must be given.")
        if inputs_embeds is not None:
            y = self.soft_embedding_norm(inputs_embeds)
        else:
            y = self.hard_embedding_norm(self.embedding(input_ids - self.vocab_offset))
        y = self.embedding_projection(y).float()
        return (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + self.eps)).to(inputs_embeds.dtype if inputs_embeds is not None else self.embedding.weight.dtype)
