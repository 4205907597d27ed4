"""Vocabulary-parallel embedding lookup: the local shard's rows for in-range ids, zeros otherwise, in one kernel
(instead of compare + masked_fill + embedding + masked_fill); the backward scatters into the local shard only
(fairseq2 ``nn/embedding.py:160-260`` ``VocabShardedEmbedding.forward``)."""

from __future__ import annotations

import os

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


class EmbeddingPush:
    """Vocabulary-parallel lookup with a token-sharded result over a symmetric arena: the rank that holds a row
    stores it into the output buffer of the rank that owns the token (one NVLink write per row, one launch, one
    barrier) instead of a zero-padded local lookup followed by a reduce-scatter that moves ``W`` times the bytes.
    The backward stages this rank's ``d(out)`` and the row owners pull the tokens they need. Every id must be a
    valid vocabulary index: a row nobody owns would keep the previous call's content."""

    SLOT = 46

    def __init__(self, arena, tokens_per_rank: int, dim: int) -> None:  # type: ignore[no-untyped-def]
        self.arena, self.rows, self.dim = arena, tokens_per_rank, dim
        n = tokens_per_rank * dim * 2
        # two forward buffers: a fast rank may push the next call's rows while a slow one still copies this call's
        self._out = [arena.alloc(n, align=16) for _ in range(2)]
        self._dout_off, dout = arena.alloc(n, align=16)
        self._dout = dout.view(torch.bfloat16).view(tokens_per_rank, dim)
        self._turn = 0

    def forward(self, ids: Tensor, shard: Tensor, lo: int) -> Tensor:
        a = self.arena
        off, buf = self._out[self._turn]
        self._turn ^= 1
        a.ext.embed_push(a.peer_ptrs, a.rank, ids, shard, lo, off, self.rows, a.wait_limit_s)
        a.barrier_next(self.SLOT)                                   # every owner's rows have landed
        return buf.view(torch.bfloat16).view(self.rows, self.dim).clone()

    def backward(self, ids: Tensor, dout: Tensor, shard_rows: int, lo: int) -> Tensor:
        a = self.arena
        self._dout.copy_(dout)
        a.barrier_next(self.SLOT)                                   # every rank has staged its token gradients
        d = a.ext.embed_pull_bwd(a.peer_ptrs, a.rank, ids, self._dout_off, shard_rows, self.dim, lo, self.rows,
                                 a.wait_limit_s)
        a.barrier_next(self.SLOT)                                   # nobody restages while a peer still reads
        return d


class _EmbedPush(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids: Tensor, shard: Tensor, lo: int, op: EmbeddingPush) -> Tensor:  # type: ignore[override]
        ctx.save_for_backward(ids)
        ctx.lo, ctx.rows, ctx.dtype, ctx.op = lo, shard.shape[0], shard.dtype, op
        return op.forward(ids, shard, lo)

    @staticmethod
    def backward(ctx, dout: Tensor):  # type: ignore[override]
        (ids,) = ctx.saved_tensors
        d = ctx.op.backward(ids, dout, ctx.rows, ctx.lo)
        return None, d.to(ctx.dtype), None, None


def _embedding_push_op(ids: Tensor, shard: Tensor, gang) -> EmbeddingPush | None:  # type: ignore[no-untyped-def]
    if not (use_kernels(ids, shard) and shard.dtype == torch.bfloat16 and shard.shape[1] % 8 == 0
            and ids.dtype == torch.int64) or os.environ.get("FAIRSEQ2_B200_TP_EMBED_PUSH", "1") == "0":
        return None
    from fairseq2_b200.parallel.tp import get_tp_context

    return get_tp_context(gang).embedding(ids.numel() // gang.size, shard.shape[1])


def embed_vocab_parallel_scatter(ids: Tensor, shard: Tensor, lo: int, gang) -> Tensor:  # type: ignore[no-untyped-def]
    """Vocabulary-parallel lookup with a sequence-parallel result: rank ``r`` of ``gang`` gets the embeddings of
    tokens ``[r * T / W, (r + 1) * T / W)`` (dimension -2 of the result). Every token's row lives on exactly one
    rank, so the sum over ranks that a reduce-scatter performs has a single non-zero term per row."""
    from fairseq2_b200.ops.tensor_parallel import reduce_scatter_seq

    if ids.shape[-1] % gang.size:
        raise ValueError(f"With sequence-parallel tensor parallelism the number of tokens ({ids.shape[-1]}) must be "
                         f"a multiple of the tensor-parallel size ({gang.size}); pad or pack the batch accordingly.")
    op = _embedding_push_op(ids, shard, gang)
    if op is not None:
        # token-major split of the flattened ids == the split of dimension -2 only when the leading dimensions are 1
        if ids.numel() == ids.shape[-1]:
            y = _EmbedPush.apply(ids.reshape(-1).contiguous(), shard, lo, op)
            return y.view(*ids.shape[:-1], ids.shape[-1] // gang.size, shard.shape[1])
    y = embed_vocab_parallel(ids, shard, lo)
    return reduce_scatter_seq(y, gang, dim=-2)
