"""Relative-position attention (cf. fairseq2 ``models/transformer/sdpa/relative.py:28-260`` and
``sdpa/shaw.py``): Transformer-XL style content/position terms with learned ``u``/``v`` biases, and
Shaw-style clipped relative key/value embeddings.

The position term is evaluated against all ``2S-1`` relative offsets and the entry for offset
``j - i`` is picked with a gather, which is the closed form of the pad-and-reshape shift."""
from __future__ import annotations

import math

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.models.transformer.attention_bias import AttentionBias, AttentionBiasCache
from fairseq2_b200.models.transformer.sdpa import SDPA, _expand_kv
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.embedding import StandardEmbedding
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.typing import DataType, Device


class RelativePositionalEncoding(Module):
    """Sinusoidal table over relative offsets ``S-1 ... -(S-1)`` (row ``p`` encodes offset ``max_seq_len-1-p``)."""

    def __init__(self, encoding_dim: int, max_seq_len: int, *, device: Device | None = None) -> None:
        super().__init__()
        if encoding_dim % 2:
            raise ValueError(f"`encoding_dim` must be even, but is {encoding_dim} instead.")
        self.encoding_dim, self.max_seq_len = encoding_dim, max_seq_len
        self.register_buffer("freqs", torch.empty((2 * max_seq_len - 1, encoding_dim), device=device,
                                                  dtype=torch.float32), persistent=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.reset_non_persistent_buffers()

    def reset_non_persistent_buffers(self) -> None:
        if self.freqs.device.type == "meta":
            return
        dev = self.freqs.device
        offsets = torch.arange(self.max_seq_len - 1, -self.max_seq_len, -1, device=dev, dtype=torch.float32)
        idx = torch.arange(0, self.encoding_dim, 2, device=dev, dtype=torch.float32)
        ang = torch.outer(offsets, torch.exp(idx * -math.log(10000.0) / self.encoding_dim))
        self.freqs[:, 0::2] = ang.sin()
        self.freqs[:, 1::2] = ang.cos()

    def forward(self, seqs: Tensor) -> Tensor:
        """``seqs``: ``(*, S, E)`` -> ``(2S-1, E)`` encodings of offsets ``S-1 ... -(S-1)``."""
        s = seqs.size(-2)
        if s > self.max_seq_len:
            raise ValueError(f"The sequence length ({s}) must not exceed the maximum sequence length "
                             f"({self.max_seq_len}).")
        return self.freqs[self.max_seq_len - s:self.max_seq_len + s - 1].type_as(seqs)


def _softmax_attend(scores: Tensor, v: Tensor, needs_weights: bool, dtype: torch.dtype) -> tuple[Tensor, Tensor | None]:
    w = torch.nan_to_num(torch.softmax(scores, dim=-1))
    out = torch.matmul(w, v.float()).transpose(-2, -3).to(dtype)
    return out, (w.to(dtype) if needs_weights else None)


class RelativePositionSDPA(SDPA):
    def __init__(self, model_dim: int, num_heads: int, pos_encoding: RelativePositionalEncoding, bias: AttentionBias, *,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(bias)
        if model_dim % num_heads:
            raise ValueError(f"`model_dim` must be a multiple of `num_heads` ({num_heads}), but is {model_dim}.")
        self.model_dim, self.num_heads = model_dim, num_heads
        self.pos_encoding = pos_encoding
        hd = model_dim // num_heads
        self.u_bias = Parameter(torch.empty((num_heads, hd), device=device, dtype=dtype))
        self.v_bias = Parameter(torch.empty((num_heads, hd), device=device, dtype=dtype))
        self.r_proj = Linear(model_dim, model_dim, bias=False, device=device, dtype=dtype)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.u_bias.device.type != "meta":
            torch.nn.init.xavier_normal_(self.u_bias)
            torch.nn.init.xavier_normal_(self.v_bias)

    def forward(self, q, q_layout, k, k_layout, v, bias_cache, *, needs_weights=False):  # type: ignore[override]
        if q_layout.packed or k_layout.packed:
            raise NotSupportedError("`RelativePositionSDPA` does not support packed batches.")
        H, D = q.shape[-2], q.shape[-1]
        k, v = _expand_kv(k, H), _expand_kv(v, H)
        qt, kt, vt = q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2)   # (N, H, S, D)
        S = kt.shape[2]
        scale = D ** -0.5
        ac = torch.matmul(qt + self.u_bias.float().unsqueeze(1), kt.transpose(-1, -2))            # content term
        r = self.r_proj(self.pos_encoding(k.transpose(1, 2)[0, 0])).view(2 * S - 1, H, D).transpose(0, 1).float()
        bd_all = torch.matmul(qt + self.v_bias.float().unsqueeze(1), r.transpose(-1, -2))         # (N, H, S, 2S-1)
        i = torch.arange(qt.shape[2], device=q.device)[:, None]
        j = torch.arange(S, device=q.device)[None, :]
        bd = bd_all.gather(-1, (S - 1 - i + j).expand(*bd_all.shape[:2], -1, -1))
        scores = (ac + bd) * scale
        b = bias_cache.get(self.bias, q_layout, k_layout, q.device, torch.float32)
        scores = scores + (b.unsqueeze(1) if b.ndim == 3 else b)
        return _softmax_attend(scores, vt, needs_weights, q.dtype)

    def extra_repr(self) -> str:
        return f"model_dim={self.model_dim}, num_heads={self.num_heads}, bias={self.bias}"


class ShawRelativePositionSDPA(SDPA):
    """Clipped relative offsets in ``[-max_left, max_right]`` index learned key (and optionally value) embeddings."""

    def __init__(self, model_dim: int, num_heads: int, max_left_rel_pos: int, bias: AttentionBias, *,
                 max_right_rel_pos: int | None = None, use_rel_pos_values: bool = False,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(bias)
        self.model_dim, self.num_heads = model_dim, num_heads
        hd = model_dim // num_heads
        self.max_left_rel_pos = max_left_rel_pos
        self.max_right_rel_pos = max_right_rel_pos if max_right_rel_pos is not None else max_left_rel_pos
        n = self.max_left_rel_pos + 1 + self.max_right_rel_pos
        self.rel_k_embed = StandardEmbedding(n, hd, init_fn=_init_shaw, device=device, dtype=dtype)
        self.rel_v_embed = StandardEmbedding(n, hd, init_fn=_init_shaw, device=device, dtype=dtype) \
            if use_rel_pos_values else None

    def _rel_indices(self, sq: int, sk: int, device: torch.device) -> Tensor:
        i = torch.arange(sq, device=device)[:, None] + (sk - sq)
        j = torch.arange(sk, device=device)[None, :]
        return (j - i).clamp(-self.max_left_rel_pos, self.max_right_rel_pos) + self.max_left_rel_pos

    def forward(self, q, q_layout, k, k_layout, v, bias_cache, *, needs_weights=False):  # type: ignore[override]
        if q_layout.packed or k_layout.packed:
            raise NotSupportedError("`ShawRelativePositionSDPA` does not support packed batches.")
        H, D = q.shape[-2], q.shape[-1]
        k, v = _expand_kv(k, H), _expand_kv(v, H)
        qt, kt, vt = q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2)
        idx = self._rel_indices(qt.shape[2], kt.shape[2], q.device)
        rel_k = self.rel_k_embed(idx).float()                                  # (Sq, Sk, D)
        scores = torch.matmul(qt, kt.transpose(-1, -2)) + torch.einsum("nhsd,std->nhst", qt, rel_k)
        scores = scores * (D ** -0.5)
        b = bias_cache.get(self.bias, q_layout, k_layout, q.device, torch.float32)
        scores = scores + (b.unsqueeze(1) if b.ndim == 3 else b)
        w = torch.nan_to_num(torch.softmax(scores, dim=-1))
        out = torch.matmul(w, vt.float())
        if self.rel_v_embed is not None:
            out = out + torch.einsum("nhst,std->nhsd", w, self.rel_v_embed(idx).float())
        return out.transpose(1, 2).to(q.dtype), (w.to(q.dtype) if needs_weights else None)


def _init_shaw(embed: StandardEmbedding) -> None:
    torch.nn.init.xavier_uniform_(embed.weight)
