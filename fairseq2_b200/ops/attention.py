"""Variable-length (packed or padded) causal GQA attention.

Sequences are described by begin offsets and lengths into the flattened token
axis, so packed batches (block-causal per document) and padded batches share
one kernel and no dense ``[S, S]`` bias is ever built. K/V heads are indexed
``h // (H / Hkv)`` inside the kernel (GQA is never materialised).
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def attention_reference(q: Tensor, k: Tensor, v: Tensor, q_begins: Tensor, q_lens: Tensor, k_begins: Tensor,
                        k_lens: Tensor, causal: bool, scale: float | None = None,
                        window: int | None = None) -> Tensor:
    """fp32 oracle. ``q``: ``[Tq, H, D]``, ``k``/``v``: ``[Tk, Hkv, D]``; returns ``[Tq, H, D]``.
    Causal masking is bottom-right aligned (query ``i`` sees keys ``j <= i + Lk - Lq``)."""
    H, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    g = H // Hkv
    for qb, ql, kb, kl in zip(q_begins.tolist(), q_lens.tolist(), k_begins.tolist(), k_lens.tolist()):
        qs = q[qb:qb + ql].float().transpose(0, 1)  # H, Lq, D
        ks = k[kb:kb + kl].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vs = v[kb:kb + kl].float().transpose(0, 1).repeat_interleave(g, dim=0)
        s = (qs @ ks.transpose(1, 2)) * scale
        i = torch.arange(ql, device=q.device)[:, None] + (kl - ql)
        j = torch.arange(kl, device=q.device)[None, :]
        if causal:
            s = s.masked_fill(j > i, float("-inf"))
        if window is not None:
            s = s.masked_fill(j <= i - window, float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p)
        out[qb:qb + ql] = (p @ vs).transpose(0, 1)
    return out.to(q.dtype)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_begins, q_lens, k_begins, k_lens, max_q, max_k, causal, scale, window,  # type: ignore[override]
                dropout_p=0.0, seed=0):
        ext = require_ext()
        out, lse = ext.attn_fwd(q, k, v, q_begins, q_lens, k_begins, k_lens, max_q, max_k, causal, scale, window,
                                dropout_p, seed)
        ctx.save_for_backward(q, k, v, out, lse, q_begins, q_lens, k_begins, k_lens)
        ctx.meta = (max_q, max_k, causal, scale, window, dropout_p, seed)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        ext = require_ext()
        q, k, v, out, lse, qb, ql, kb, kl = ctx.saved_tensors
        max_q, max_k, causal, scale, window, dropout_p, seed = ctx.meta
        dq, dk, dv = ext.attn_bwd(dout.contiguous(), q, k, v, out, lse, qb, ql, kb, kl, max_q, max_k, causal, scale,
                                  window, dropout_p, seed)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None, None, None


def varlen_attention(q: Tensor, k: Tensor, v: Tensor, q_begins: Tensor, q_lens: Tensor, k_begins: Tensor,
                     k_lens: Tensor, max_q: int, max_k: int, *, causal: bool = True, scale: float | None = None,
                     window: int | None = None, dropout_p: float = 0.0, seed: int | None = None) -> Tensor:
    """``dropout_p``: dropout on the attention probabilities inside the kernels (the mask is a hash of ``seed``, the
    head and the token pair, evaluated again in the backward pass; nothing is stored). ``seed`` defaults to a draw
    from the CPU generator, so ``torch.manual_seed`` makes runs repeatable. Without the kernels the reference
    formulation is used and dropout is not supported there."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    windowed = window is not None and window > 0
    if (use_kernels(q) and q.dtype == torch.bfloat16 and D in (64, 128) and (not windowed or (causal and D == 128))
            and q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and not (windowed and dropout_p > 0.0)):
        if dropout_p > 0.0 and seed is None:
            seed = int(torch.randint(0, 2**62, (1,), device="cpu"))
        return _AttnFn.apply(q, k, v, q_begins, q_lens, k_begins, k_lens, max_q, max_k, causal, scale,
                             window if windowed else 0, float(dropout_p), int(seed or 0))
    if dropout_p > 0.0:
        raise NotImplementedError("Attention dropout needs the CUDA kernels (bf16, head_dim 64 or 128, no window).")
    return attention_reference(q, k, v, q_begins, q_lens, k_begins, k_lens, causal, scale, window)


class _QKVRopeAttnFn(torch.autograd.Function):
    """Self-attention over a merged ``[T, H + 2·Hkv, D]`` projection output:
    in-place RoPE on the q and k heads, varlen attention reading strided views,
    and a backward that writes dq|dk|dv into one merged buffer so the
    projection's dgrad/wgrad GEMMs consume it without a concat."""

    @staticmethod
    def forward(ctx, qkv, freqs, positions, begins, lens, max_len, causal, scale, H, Hkv, has_padding, window=0,  # type: ignore[override]
                dropout_p=0.0, seed=0):
        ext = require_ext()
        if freqs is not None:
            # The producer of `qkv` (the merged projection) does not need its own
            # output in backward, so rotating it in place is safe; the raw kernel
            # call bypasses autograd's version counters by construction.
            ext.rope_inplace(qkv[:, : H + Hkv], freqs, positions, False)
        q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
        out, lse = ext.attn_fwd(q, k, v, begins, lens, begins, lens, max_len, max_len, causal, scale, window,
                                dropout_p, seed)
        ctx.save_for_backward(qkv, out, lse, begins, lens, freqs, positions)
        ctx.meta = (max_len, causal, scale, H, Hkv, has_padding, window, dropout_p, seed)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        ext = require_ext()
        qkv, out, lse, begins, lens, freqs, positions = ctx.saved_tensors
        max_len, causal, scale, H, Hkv, has_padding, window, dropout_p, seed = ctx.meta
        q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
        # rows outside every sequence are never written by the kernels: they must read as zero gradients
        dqkv = torch.zeros_like(qkv) if has_padding else torch.empty_like(qkv)
        ext.attn_bwd_out(dout.contiguous(), q, k, v, out, lse, begins, lens, begins, lens, max_len, max_len, causal,
                         scale, dqkv[:, :H], dqkv[:, H:H + Hkv], dqkv[:, H + Hkv:], window, dropout_p, seed)
        if freqs is not None:
            ext.rope_inplace(dqkv[:, : H + Hkv], freqs, positions, True)
        return dqkv, None, None, None, None, None, None, None, None, None, None, None, None, None


def qkv_rope_attention(qkv: Tensor, freqs: Tensor | None, positions: Tensor | None, begins: Tensor, lens: Tensor,
                       max_len: int, *, num_heads: int, num_kv_heads: int, causal: bool = True,
                       scale: float | None = None, has_padding: bool = True, window: int | None = None,
                       dropout_p: float = 0.0, seed: int | None = None) -> Tensor:
    """``qkv``: contiguous bf16 ``[T, H + 2·Hkv, D]`` (modified in place). Returns ``[T, H, D]``. ``window``
    (causal, head_dim 128 only): every query sees at most that many most recent keys, itself included.
    ``dropout_p`` / ``seed``: see :func:`varlen_attention` (not together with a window)."""
    D = qkv.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if dropout_p > 0.0 and seed is None:
        seed = int(torch.randint(0, 2**62, (1,), device="cpu"))
    return _QKVRopeAttnFn.apply(qkv, freqs, positions, begins, lens, max_len, causal, scale, num_heads, num_kv_heads,
                                has_padding, window or 0, float(dropout_p), int(seed or 0))
