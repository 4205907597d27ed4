"""Attention bias descriptions (cf. fairseq2 ``models/transformer/attention_bias.py``:
``IdentityBias`` :22, ``CausalAttentionBias`` :52, ``ChunkedAttentionBias``,
``ALiBiAttentionBias``, ``materialize_attention_bias`` :235-326, cache :346).

A bias object only *describes* the mask. The varlen attention kernel evaluates
identity/causal/sliding-window masks (and per-document block structure of
packed batches) from sequence offsets, so a dense tensor is materialised only
for the bias kinds the kernel does not know (ALiBi, chunked) and for the naive
SDPA oracle.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod

import torch
from torch import Tensor

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.typing import DataType, Device


class AttentionBias(ABC):
    @abstractmethod
    def materialize(self, q_len: int, k_len: int, device: Device, dtype: DataType) -> Tensor:
        """Additive ``([H], q_len, k_len)`` bias for ONE sequence; queries are
        bottom-right aligned with keys."""


class IdentityBias(AttentionBias):
    def materialize(self, q_len: int, k_len: int, device: Device, dtype: DataType) -> Tensor:
        return torch.zeros((q_len, k_len), device=device, dtype=dtype)

    def __repr__(self) -> str:
        return "IdentityBias()"


class CausalAttentionBias(AttentionBias):
    def __init__(self, *, attn_window_len: int | None = None) -> None:
        self.attn_window_len = attn_window_len

    def materialize(self, q_len: int, k_len: int, device: Device, dtype: DataType) -> Tensor:
        i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
        j = torch.arange(k_len, device=device)[None, :]
        dead = j > i
        if self.attn_window_len is not None:
            dead |= j <= i - self.attn_window_len
        return torch.zeros((q_len, k_len), device=device, dtype=dtype).masked_fill_(dead, float("-inf"))

    def __repr__(self) -> str:
        return f"CausalAttentionBias(attn_window_len={self.attn_window_len})"


class ChunkedAttentionBias(AttentionBias):
    """Causal attention restricted to chunks of ``attn_chunk_size`` positions (LLaMA-4)."""

    def __init__(self, *, attn_chunk_size: int) -> None:
        self.attn_chunk_size = attn_chunk_size

    def materialize(self, q_len: int, k_len: int, device: Device, dtype: DataType) -> Tensor:
        i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
        j = torch.arange(k_len, device=device)[None, :]
        dead = (j > i) | ((i // self.attn_chunk_size) != (j // self.attn_chunk_size))
        return torch.zeros((q_len, k_len), device=device, dtype=dtype).masked_fill_(dead, float("-inf"))

    def __repr__(self) -> str:
        return f"ChunkedAttentionBias(attn_chunk_size={self.attn_chunk_size})"


class ALiBiAttentionBias(AttentionBias):
    def __init__(self, num_heads: int) -> None:
        self.num_heads = num_heads

    def materialize(self, q_len: int, k_len: int, device: Device, dtype: DataType) -> Tensor:
        n = self.num_heads
        p = 2 ** math.floor(math.log2(n))
        base = 2.0 ** (-8.0 / p)
        slopes = torch.pow(base, torch.arange(1, 1 + p, device=device, dtype=torch.float32))
        if p != n:
            base2 = 2.0 ** (-4.0 / p)
            extra = torch.pow(base2, torch.arange(1, 1 + 2 * (n - p), 2, device=device, dtype=torch.float32))
            slopes = torch.cat([slopes, extra])
        i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
        j = torch.arange(k_len, device=device)[None, :]
        dist = (j - i).float().clamp(max=0)  # <= 0 for visible keys
        bias = slopes[:, None, None] * dist[None]
        bias = bias.masked_fill((j > i)[None], float("-inf"))
        return bias.to(dtype)

    def __repr__(self) -> str:
        return f"ALiBiAttentionBias(num_heads={self.num_heads})"


def materialize_attention_bias(bias: AttentionBias, q_layout: BatchLayout, k_layout: BatchLayout, device: Device,
                               dtype: DataType) -> Tensor:
    """Dense additive bias for a whole batch.

    Padded batches: ``(N, [H], S, S_kv)`` with key padding masked. Packed
    batches: ``([H], T, T_kv)`` block-diagonal over documents.
    """
    neg = float("-inf")
    if q_layout.packed != k_layout.packed:
        raise ValueError("`q_layout` and `k_layout` must be both packed or both unpacked.")
    if q_layout.packed:
        tq, tk = q_layout.width, k_layout.width
        blocks = []
        for ql, kl in zip(q_layout.seq_lens, k_layout.seq_lens):
            blocks.append(bias.materialize(ql, kl, device, dtype))
        lead = blocks[0].shape[:-2] if blocks else ()
        full = torch.full((*lead, tq, tk), neg, device=device, dtype=dtype)
        for b, qb, kb, ql, kl in zip(blocks, q_layout.seq_begin_indices, k_layout.seq_begin_indices,
                                     q_layout.seq_lens, k_layout.seq_lens):
            full[..., qb:qb + ql, kb:kb + kl] = b
        return full
    n = len(q_layout.seq_lens)
    sq, sk = q_layout.width, k_layout.width
    outs = []
    for ql, kl in zip(q_layout.seq_lens, k_layout.seq_lens):
        b = bias.materialize(ql, kl, device, dtype)
        lead = b.shape[:-2]
        full = torch.full((*lead, sq, sk), neg, device=device, dtype=dtype)
        full[..., :ql, :kl] = b
        if ql < sq:
            full[..., ql:, :1] = 0.0  # padded query rows attend to something finite
        outs.append(full)
    return torch.stack(outs, dim=0) if n else torch.empty((0, sq, sk), device=device, dtype=dtype)


class AttentionBiasCache:
    """Per-forward memo of materialised biases keyed by (bias, layouts)."""

    def __init__(self) -> None:
        self._data: dict[tuple[int, int, int, str], Tensor] = {}

    def get(self, bias: AttentionBias, q_layout: BatchLayout, k_layout: BatchLayout, device: Device,
            dtype: DataType) -> Tensor:
        key = (id(bias), id(q_layout), id(k_layout), str(dtype))
        t = self._data.get(key)
        if t is None:
            t = materialize_attention_bias(bias, q_layout, k_layout, device, dtype)
            self._data[key] = t
        return t

    def clear(self) -> None:
        self._data.clear()
