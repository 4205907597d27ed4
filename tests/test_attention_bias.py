"""Attention biases against explicit masks: causal (bottom-right aligned), sliding window, chunked, ALiBi, and their
padded / packed batch forms (cf. fairseq2 ``models/transformer/attention_bias.py:52-142,285-324``)."""
from __future__ import annotations

import math

import torch

from fairseq2_b200.models.transformer.attention_bias import (ALiBiAttentionBias, CausalAttentionBias,
                                                             ChunkedAttentionBias, IdentityBias,
                                                             materialize_attention_bias)
from fairseq2_b200.nn import BatchLayout

CPU, F32 = torch.device("cpu"), torch.float32


def _visible(bias: torch.Tensor) -> list[list[int]]:
    return (bias > float("-inf")).int().tolist()


def test_causal_is_bottom_right_aligned() -> None:
    assert _visible(CausalAttentionBias().materialize(3, 3, CPU, F32)) == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    # two new queries against five keys (incremental decoding): the last query sees everything
    assert _visible(CausalAttentionBias().materialize(2, 5, CPU, F32)) == [[1, 1, 1, 1, 0], [1, 1, 1, 1, 1]]


def test_sliding_window_and_chunks() -> None:
    win = _visible(CausalAttentionBias(attn_window_len=2).materialize(4, 4, CPU, F32))
    assert win == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]
    chunk = _visible(ChunkedAttentionBias(attn_chunk_size=2).materialize(4, 4, CPU, F32))
    assert chunk == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 0, 1, 0], [0, 0, 1, 1]]


def test_alibi_slopes() -> None:
    b = ALiBiAttentionBias(4).materialize(3, 3, CPU, F32)
    assert b.shape == (4, 3, 3)
    for h in range(4):
        slope = 2.0 ** (-8.0 * (h + 1) / 4)
        assert float(b[h, 2, 0]) == -2 * slope and float(b[h, 2, 2]) == 0.0 and math.isinf(float(b[h, 0, 1]))
    assert ALiBiAttentionBias(6).materialize(2, 2, CPU, F32).shape[0] == 6      # non power of two head counts


def test_batch_forms() -> None:
    x = torch.zeros(2, 3)
    padded = materialize_attention_bias(CausalAttentionBias(), BatchLayout.of(x, [3, 2]), BatchLayout.of(x, [3, 2]),
                                        CPU, F32)
    assert padded.shape == (2, 3, 3)
    assert _visible(padded[1])[:2] == [[1, 0, 0], [1, 1, 0]]                     # the padded key column is masked
    assert torch.isfinite(padded[1, 2]).any()                                     # padded query rows stay finite
    p = torch.zeros(5)
    layout = BatchLayout.of(p, [2, 3], packed=True)
    packed = materialize_attention_bias(CausalAttentionBias(), layout, layout, CPU, F32)
    assert _visible(packed) == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 1, 1, 1]]
    ident = materialize_attention_bias(IdentityBias(), layout, layout, CPU, F32)
    assert _visible(ident) == [[1, 1, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 1, 1], [0, 0, 1, 1, 1], [0, 0, 1, 1, 1]]
