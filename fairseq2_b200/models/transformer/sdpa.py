"""Scaled dot-product attention variants.

fairseq2 ships ``TorchSDPA``, ``NaiveSDPA``, ``Flash2SDPA``, ``Flash3SDPA``,
``SoftCappedSDPA`` and relative-position variants (``models/transformer/sdpa/*``).
Here the default is :class:`VarlenSDPA`, backed by the in-tree sm_100a kernel
that handles padded and packed layouts, GQA and causal/identity biases
natively. :class:`NaiveSDPA` (fp32 matmul/softmax with a dense bias) is the
oracle and the fallback for bias kinds the kernel does not evaluate;
:class:`TorchSDPA` wraps ``F.scaled_dot_product_attention``.

Shapes: ``q`` ``([N], S, H, D)``, ``k``/``v`` ``([N], S_kv, H_kv, D)``.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Callable

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module

from fairseq2_b200.models.transformer.attention_bias import (AttentionBias, AttentionBiasCache, CausalAttentionBias,
                                                              IdentityBias, materialize_attention_bias)
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.ops._ext import use_kernels
from fairseq2_b200.ops.attention import varlen_attention


class SDPA(Module, ABC):
    def __init__(self, bias: AttentionBias) -> None:
        super().__init__()
        self.bias = bias

    @abstractmethod
    def forward(self, q: Tensor, q_layout: BatchLayout, k: Tensor, k_layout: BatchLayout, v: Tensor,
                bias_cache: AttentionBiasCache, *, needs_weights: bool = False) -> tuple[Tensor, Tensor | None]: ...


def _expand_kv(k: Tensor, num_heads: int) -> Tensor:
    hkv = k.shape[-2]
    if hkv == num_heads:
        return k
    return k.repeat_interleave(num_heads // hkv, dim=-2)


class NaiveSDPA(SDPA):
    """fp32 reference: explicit scores, dense bias, softmax, weighted sum."""

    def __init__(self, bias: AttentionBias, *, dropout_p: float = 0.0, soft_cap: float | None = None) -> None:
        super().__init__(bias)
        self.dropout_p = dropout_p
        self.soft_cap = soft_cap

    def forward(self, q, q_layout, k, k_layout, v, bias_cache, *, needs_weights=False):  # type: ignore[override]
        H = q.shape[-2]
        k, v = _expand_kv(k, H), _expand_kv(v, H)
        qt, kt, vt = q.transpose(-2, -3), k.transpose(-2, -3), v.transpose(-2, -3)  # ([N], H, S, D)
        w = torch.matmul(qt.float(), kt.float().transpose(-1, -2)) * (q.shape[-1] ** -0.5)
        if self.soft_cap is not None:
            w = torch.tanh(w / self.soft_cap) * self.soft_cap
        b = bias_cache.get(self.bias, q_layout, k_layout, q.device, torch.float32)
        if not q_layout.packed and b.ndim == 3:
            b = b.unsqueeze(1)
        w = torch.softmax(w + b, dim=-1)
        w = torch.nan_to_num(w)
        if self.training and self.dropout_p > 0.0:
            w = F.dropout(w, self.dropout_p)
        out = torch.matmul(w, vt.float()).transpose(-2, -3).to(q.dtype)
        return out, (w.to(q.dtype) if needs_weights else None)


class SoftCappedSDPA(NaiveSDPA):
    """``tanh(s / cap) * cap`` logit capping (Gemma)."""

    def __init__(self, bias: AttentionBias, *, soft_cap: float, dropout_p: float = 0.0) -> None:
        super().__init__(bias, dropout_p=dropout_p, soft_cap=soft_cap)


class TorchSDPA(SDPA):
    def __init__(self, bias: AttentionBias, *, dropout_p: float = 0.0) -> None:
        super().__init__(bias)
        self.dropout_p = dropout_p

    def forward(self, q, q_layout, k, k_layout, v, bias_cache, *, needs_weights=False):  # type: ignore[override]
        if needs_weights or q_layout.packed:
            return NaiveSDPA(self.bias, dropout_p=self.dropout_p).forward(
                q, q_layout, k, k_layout, v, bias_cache, needs_weights=needs_weights)
        H = q.shape[-2]
        k, v = _expand_kv(k, H), _expand_kv(v, H)
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        full = not q_layout.padded and not k_layout.padded
        p = self.dropout_p if self.training else 0.0
        if full and isinstance(self.bias, IdentityBias):
            out = F.scaled_dot_product_attention(qt, kt, vt, dropout_p=p)
        elif full and isinstance(self.bias, CausalAttentionBias) and self.bias.attn_window_len is None \
                and q.shape[1] == k.shape[1]:
            out = F.scaled_dot_product_attention(qt, kt, vt, dropout_p=p, is_causal=True)
        else:
            b = bias_cache.get(self.bias, q_layout, k_layout, q.device, q.dtype)
            if b.ndim == 3:
                b = b.unsqueeze(1)
            out = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=b, dropout_p=p)
        return out.transpose(1, 2), None


class VarlenSDPA(SDPA):
    """Default SDPA: in-tree varlen flash attention (identity / causal /
    sliding-window biases); anything else is routed to :class:`NaiveSDPA`."""

    def __init__(self, bias: AttentionBias, *, dropout_p: float = 0.0) -> None:
        super().__init__(bias)
        self.dropout_p = dropout_p
        self._naive = NaiveSDPA(bias, dropout_p=dropout_p)

    def forward(self, q, q_layout, k, k_layout, v, bias_cache, *, needs_weights=False):  # type: ignore[override]
        supported = isinstance(self.bias, (IdentityBias, CausalAttentionBias))
        drop = self.dropout_p if self.training else 0.0
        kernel_dropout = (drop == 0.0 or (use_kernels(q) and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)
                                          and getattr(self.bias, "attn_window_len", None) is None))
        if needs_weights or not supported or not kernel_dropout:
            return self._naive(q, q_layout, k, k_layout, v, bias_cache, needs_weights=needs_weights)
        causal = isinstance(self.bias, CausalAttentionBias)
        window = self.bias.attn_window_len if causal else None
        packed = q_layout.packed
        if packed:
            q2, k2, v2 = q, k, v
        else:
            q2, k2, v2 = q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1)
        out = varlen_attention(q2, k2, v2, q_layout.seq_begin_indices_pt[:-1], q_layout.seq_lens_pt,
                               k_layout.seq_begin_indices_pt[:-1], k_layout.seq_lens_pt, q_layout.max_seq_len,
                               k_layout.max_seq_len, causal=causal, window=window, dropout_p=drop)
        if not packed:
            out = out.view(q.shape)
        return out, None


Flash2SDPA = VarlenSDPA  # name kept for configs that ask for "flash2"
Flash3SDPA = VarlenSDPA

_default_factory: Callable[..., SDPA] = VarlenSDPA


def set_default_sdpa_factory(factory: Callable[..., SDPA]) -> None:
    global _default_factory
    _default_factory = factory


def get_default_sdpa_factory() -> Callable[..., SDPA]:
    return _default_factory


def create_default_sdpa(bias: AttentionBias, *, dropout_p: float = 0.0) -> SDPA:
    return _default_factory(bias, dropout_p=dropout_p)


def sdpa_factory_by_name(name: str) -> Callable[..., SDPA]:
    table: dict[str, Callable[..., SDPA]] = {"torch": TorchSDPA, "torch_math": NaiveSDPA, "naive": NaiveSDPA,
                                             "flash2": VarlenSDPA, "flash3": VarlenSDPA, "varlen": VarlenSDPA,
                                             "b200": VarlenSDPA}
    try:
        return table[name]
    except KeyError:
        raise ValueError(f"`name` must be one of {sorted(table)}, but is '{name}' instead.") from None
