"""Vocabulary-parallel embedding lookup: the local shard's rows for in-range ids, zeros otherwise, in one kernel
(instead of compare + masked_fill + embedding + masked_fill); the backward scatters into the local shard only
(fairseq2 ``nn/embedding.py:160-260`` ``VocabShardedEmbedding.forward``)."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def embed_vocab_parallel_reference(ids: Tensor, shard: Tensor, lo: int) -> Tensor:
    hi = lo + shard.shape[0]
    oob = (ids < lo) | (ids >= hi)
    y = F.embedding((ids - lo).masked_fill(oob, 0), shard)
    return y.masked_fill(oob.unsqueeze(-1), 0.0)


class _EmbedVocabParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids: Tensor, shard: Tensor, lo: int) -> Tensor:  # type: ignore[override]
        ctx.save_for_backward(ids)
        ctx.lo, ctx.rows, ctx.dtype = lo, shard.shape[0], shard.dtype
        return require_ext().embed_vocab_parallel_fwd(ids, shard, lo, 1.0)

    @staticmethod
    def backward(ctx, dout: Tensor):  # type: ignore[override]
        (ids,) = ctx.saved_tensors
        d = require_ext().embed_vocab_parallel_bwd(ids, dout.contiguous(), ctx.rows, ctx.lo, 1.0)
        return None, d.to(ctx.dtype), None


def embed_vocab_parallel(ids: Tensor, shard: Tensor, lo: int) -> Tensor:
    """``ids`` int64 of any shape, ``shard`` ``[rows, D]`` holding vocabulary rows ``[lo, lo + rows)`` ->
    ``[*ids.shape, D]``; summing the result over the ranks of the vocabulary-parallel group gives the full lookup."""
    if use_kernels(ids, shard) and shard.dtype == torch.bfloat16 and shard.shape[1] % 8 == 0 and ids.dtype == torch.int64:
        return _EmbedVocabParallel.apply(ids.contiguous(), shard, lo)
    return embed_vocab_parallel_reference(ids, shard, lo)


def embed_vocab_parallel_scatter(ids: Tensor, shard: Tensor, lo: int, gang) -> Tensor:  # type: ignore[no-untyped-def]
    """Vocabulary-parallel lookup with a sequence-parallel result: rank ``r`` of ``gang`` gets the embeddings of
    tokens ``[r * T / W, (r + 1) * T / W)`` (dimension -2 of the result). Every token's row lives on exactly one
    rank, so the sum over ranks that a reduce-scatter performs has a single non-zero term per row."""
    from fairseq2_b200.ops.tensor_parallel import reduce_scatter_seq

    if ids.shape[-1] % gang.size:
        raise ValueError(f"With sequence-parallel tensor parallelism the number of tokens ({ids.shape[-1]}) must be "
                         f"a multiple of the tensor-parallel size ({gang.size}); pad or pack the batch accordingly.")
    y = embed_vocab_parallel(ids, shard, lo)
    return reduce_scatter_seq(y, gang, dim=-2)
