"""Tensor parallelism with sequence-parallel activations: build-time switch and the per-gang registry of the fused
all-gather / reduce-scatter GEMM operators.

``with sequence_parallel():`` around a model factory makes the tensor-parallel layers it creates sequence parallel:
between the blocks every rank holds ``T / W`` tokens of the residual stream, the column-parallel projections
all-gather the tokens inside their GEMM and the row-parallel projections reduce-scatter their output from the GEMM
epilogue (fairseq2 has no such mode: its column/row layers all-reduce full ``[T, D]`` activations,
``nn/projection.py:281-288,519-527``). Incremental decoding keeps the default (tokens replicated).

On CUDA the projections look their operators up here: one symmetric arena per tensor-parallel gang, one
``SequenceParallelLinears`` per ``(tokens per rank, model dim)``. Where the arena cannot be had (CPU ranks, no peer
access, a shape the kernels do not cover) the layers fall back to the gang's collectives.
"""
from __future__ import annotations

import os
import threading
from contextlib import contextmanager
from typing import Any, Iterator

import torch
from torch import Tensor

from fairseq2_b200.gang import Gang
from fairseq2_b200.logging import log

_flag = threading.local()


def sequence_parallel_enabled() -> bool:
    return bool(getattr(_flag, "on", False))


@contextmanager
def sequence_parallel(enabled: bool = True) -> Iterator[None]:
    old = sequence_parallel_enabled()
    _flag.on = enabled
    try:
        yield
    finally:
        _flag.on = old


class TPContext:
    """Fused tensor-parallel operators of one gang (created on first use)."""

    def __init__(self, gang: Gang) -> None:
        self.gang = gang
        self.arena: Any = None
        self._ops: dict[tuple[int, int], Any] = {}
        self._tried = False

    def _ensure_arena(self) -> Any:
        if self._tried:
            return self.arena
        self._tried = True
        if os.environ.get("FAIRSEQ2_B200_TP_FUSED", "1") == "0":
            return None
        from fairseq2_b200.parallel.symm import SymmetricArena, symmetric_memory_available

        if not symmetric_memory_available(self.gang):
            return None
        mb = int(os.environ.get("FAIRSEQ2_B200_TP_ARENA_MB", "1536"))
        torch.cuda.empty_cache()              # symmetric memory is allocated outside the caching allocator
        try:
            wait = float(os.environ.get("FAIRSEQ2_B200_WAIT_LIMIT_S", "120"))
            self.arena = SymmetricArena(self.gang, mb << 20, wait_limit_s=wait)  # type: ignore[arg-type]
        except Exception as ex:  # noqa: BLE001 - no peer access: the layers use the gang's collectives
            log.warning("Symmetric memory is not usable for tensor parallelism ({}); using gang collectives.", ex)
            self.arena = None
        return self.arena

    def prepare(self) -> bool:
        """Creates the arena now (a collective call: every rank of the gang must make it) instead of inside the
        first forward pass, e.g. while memory is still plentiful; returns whether the fused operators are usable."""
        return self._ensure_arena() is not None

    def linears(self, like: Tensor, rows: int, dim: int) -> Any | None:
        """The fused operator set for token shards ``[rows, dim]`` (``like``: a bf16 CUDA tensor of the call), or
        ``None`` when the fused kernels do not cover the case."""
        if not (like.is_cuda and like.dtype == torch.bfloat16 and like.ndim == 2):
            return None
        if rows <= 0 or rows % 128 or dim % 64:
            return None
        key = (rows, dim)
        ops = self._ops.get(key)
        if ops is None:
            arena = self._ensure_arena()
            if arena is None:
                return None
            from fairseq2_b200.ops.fused_collective import SequenceParallelLinears

            try:
                ops = SequenceParallelLinears(arena, rows, dim)
            except MemoryError as ex:
                log.warning("The tensor-parallel arena is too small for {} x {} token shards ({}); set "
                            "FAIRSEQ2_B200_TP_ARENA_MB.", rows, dim, ex)
                self._ops[key] = False
                return None
            self._ops[key] = ops
        return ops or None


    def embedding(self, rows: int, dim: int) -> Any | None:
        """The row-push operator of the vocabulary-parallel embedding for ``rows`` tokens per rank."""
        if rows <= 0 or dim % 8:
            return None
        key = (-rows, dim)
        op = self._ops.get(key)
        if op is None:
            arena = self._ensure_arena()
            if arena is None:
                return None
            from fairseq2_b200.ops.embedding import EmbeddingPush

            try:
                op = EmbeddingPush(arena, rows, dim)
            except MemoryError:
                self._ops[key] = False
                return None
            self._ops[key] = op
        return op or None


_contexts: dict[int, TPContext] = {}


def get_tp_context(gang: Gang) -> TPContext:
    ctx = _contexts.get(id(gang))
    if ctx is None:
        ctx = _contexts[id(gang)] = TPContext(gang)
    return ctx
