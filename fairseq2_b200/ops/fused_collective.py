"""Compute + collective fused into one kernel over NVLink peer memory.

``FusedGemmReduceScatter`` is the row-parallel linear layer of tensor parallelism with a sequence-parallel
output: every rank multiplies its slice of the activations by its slice of the weight and the partial products
must be summed over ranks, rank ``r`` keeping rows ``[r·M/W, (r+1)·M/W)``. Instead of a GEMM followed by a
reduce-scatter, the tcgen05 GEMM's epilogue adds every fp32 accumulator tile straight into the memory of the
rank that owns its rows (``red.global.add.v4.f32`` through the peer mapping), so the NVLink transfer of tile
``i`` overlaps the tensor-core work of tile ``i + 1`` and the full ``[M, N]`` partial product never exists.

The destination buffers live in a symmetric arena and alternate between two slots: a slot is zeroed one call
ahead, so each call needs a single cross-rank barrier (after the kernel, when all additions have landed).
"""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.ops.gemm import gemm
from fairseq2_b200.parallel.symm import SymmetricArena


def gemm_reduce_scatter_reference(x_parts: list[Tensor], w_parts: list[Tensor], rank: int) -> Tensor:
    """fp32 oracle: ``sum_r x_r @ w_rᵀ`` restricted to the rows that ``rank`` owns."""
    full = sum(x.float() @ w.float().t() for x, w in zip(x_parts, w_parts))
    rows = full.shape[0] // len(x_parts)
    return full[rank * rows:(rank + 1) * rows]


class FusedGemmReduceScatter:
    """Row-parallel linear layer fused with its reduce-scatter: ``out[rank] = (sum_r x_r @ w_r^T)[rows of rank]``.

    The GEMM epilogue sends every output tile over NVLink to the rank that owns its rows while the next tile is on
    the tensor cores. ``mode="scatter"`` (default): tiles are rounded to bf16 and written with plain stores into this
    rank's slice of the owner's ``[world, rows, N]`` buffer; after a barrier the owner sums its slices in fp32 (the
    numerics of a bf16 reduce-scatter, deterministic, 2 bytes per element on the wire). ``mode="red"``: fp32 tiles
    are summed in place in the owner's buffer with ``red.global.add`` (no rounding of the partial products, 4 bytes
    per element, summation order not fixed).
    """

    #: barrier slot inside the arena's flag page reserved for this operator family
    SLOT = 40

    def __init__(self, arena: SymmetricArena, max_rows_per_rank: int, out_dim: int, *, mode: str = "scatter",
                 out_dtype: torch.dtype = torch.bfloat16) -> None:
        if mode not in ("scatter", "red"):
            raise ValueError(f"`mode` must be 'scatter' or 'red', but is '{mode}' instead.")
        self.arena, self.mode, self.out_dtype = arena, mode, out_dtype
        self.max_rows, self.out_dim = max_rows_per_rank, out_dim
        self._which = 0
        if mode == "red":
            self._slots = [arena.alloc_tensor(max_rows_per_rank * out_dim, torch.float32) for _ in range(2)]
            for _, buf in self._slots:
                buf.zero_()
            # every rank's slots are zero before anyone adds into them
            arena.barrier_next(self.SLOT)
        else:
            self._slots = [arena.alloc_tensor(arena.world * max_rows_per_rank * out_dim, torch.bfloat16)
                           for _ in range(2)]

    def __call__(self, x: Tensor, weight: Tensor, *, weight_kn: bool = False) -> Tensor:
        """``x``: bf16 ``[M, K_local]``, ``weight``: bf16 ``[N, K_local]`` (or ``[K_local, N]`` with ``weight_kn``,
        "scatter" mode only) -> ``[M / world, N]``. In "red" mode the result is an fp32 view into the arena that
        stays valid until the call after the next one."""
        arena = self.arena
        if weight_kn and self.mode != "scatter":
            raise ValueError("`weight_kn` needs mode='scatter'.")
        M, N = x.shape[0], weight.shape[1 if weight_kn else 0]
        if M % arena.world:
            raise ValueError(f"The number of rows ({M}) must be a multiple of the world size ({arena.world}).")
        rows = M // arena.world
        if rows > self.max_rows or N != self.out_dim:
            raise ValueError("The operands exceed the shapes this operator was created for.")
        off, buf = self._slots[self._which]
        nxt_off, nxt = self._slots[self._which ^ 1]
        self._which ^= 1
        if self.mode == "red":
            arena.ext.gemm_reduce_scatter(x.contiguous(), weight.contiguous(), arena.peer_ptrs, off, rows)
            nxt.zero_()                       # the other slot is free again: its last reader ran before this call
            arena.barrier_next(self.SLOT)     # all ranks' additions have landed (and their next slots are zero)
            return buf[: rows * N].view(rows, N)
        # two slots alternate: a rank passes the barrier of call k + 1 only after its own sum of call k, so the
        # slot written by call k + 2 is no longer being read by anyone
        arena.ext.gemm_scatter(x.contiguous(), weight.contiguous(), arena.peer_ptrs, arena.rank, off, rows, weight_kn)
        arena.barrier_next(self.SLOT)         # every rank's tiles for my rows have landed
        out = torch.empty((rows, N), device=x.device, dtype=self.out_dtype)
        arena.ext.reduce_slices(buf[: arena.world * rows * N].view(arena.world, rows * N), out)
        return out


class FusedAllGatherGemm:
    """All-gather of one GEMM operand fused into the tcgen05 GEMM.

    ``gather="a"`` is the column-parallel linear layer with a sequence-parallel input: every rank holds
    ``[M / W, K]`` rows of the activations and ``[N_local, K]`` of the weight; ``gather="b"`` is the FSDP
    unshard: every rank holds ``[N / W, K]`` rows of the weight and all of the activations.

    A few CTAs of the GEMM grid copy the peers' shards over NVLink into local memory -- each byte crosses once,
    own shard (already in place) first, then the peers in ring order -- and raise one flag per tile-height block; the TMA producers
    of the compute CTAs wait for the flag of the block they need. The GEMM therefore starts at once on local data
    and the remaining transfers overlap tensor-core work inside the same kernel.

    Usage: write the local shard into ``self.shard`` (a view into the symmetric arena), then call the operator.
    """

    SLOT = 42

    def __init__(self, arena: SymmetricArena, rows_per_rank: int, k: int, *, gather: str = "a",
                 num_copy_ctas: int = 8) -> None:
        if gather not in ("a", "b"):
            raise ValueError("`gather` must be 'a' or 'b'.")
        blk = 256 if gather == "b" else 128
        if rows_per_rank % blk:
            raise ValueError(f"`rows_per_rank` must be a multiple of {blk} for gather='{gather}'.")
        self.arena, self.rows, self.k, self.gather_b = arena, rows_per_rank, k, gather == "b"
        self.ncopy = num_copy_ctas
        # the own shard lives at its final place inside the gathered operand, so it is never copied
        self._gathered_off, gathered = arena.alloc(arena.world * rows_per_rank * k * 2, align=1024)
        self.shard = gathered.view(torch.bfloat16).view(arena.world, rows_per_rank, k)[arena.rank]
        self._shard_off = -16
        nblocks = arena.world * rows_per_rank // blk
        self._flags_off, flags = arena.alloc(4 * nblocks, align=16)
        flags.zero_()
        self._epoch = 0
        self._bar_epoch = 0

    @property
    def gathered(self) -> Tensor:
        """The assembled operand ``[world * rows, k]`` (valid after a call until the shard is rewritten)."""
        a = self.arena
        n = a.world * self.rows * self.k * 2
        return a.buf[self._gathered_off: self._gathered_off + n].view(torch.bfloat16).view(a.world * self.rows, self.k)

    def __call__(self, other: Tensor, out: Tensor | None = None, *, other_kn: bool = False) -> Tensor:
        """``other``: the local operand ``[N, k]`` (gather="a"; ``[k, N]`` with ``other_kn``) or ``[M, k]``
        (gather="b")."""
        a = self.arena
        W = a.world
        if self.gather_b:
            M, N = other.shape[0], self.rows * W
        else:
            M, N = self.rows * W, other.shape[1 if other_kn else 0]
        if out is None:
            out = torch.empty((M, N), device=other.device, dtype=torch.bfloat16)
        # every rank has written its shard (and finished reading the shards of the previous call)
        a.barrier_next(self.SLOT)
        self._epoch += 1
        a.ext.gemm_allgather(a.peer_ptrs, a.rank, self._shard_off, self.rows, other.contiguous(), self._gathered_off,
                             self._flags_off, self._epoch, self.gather_b, out, self.ncopy, other_kn)
        # nobody may overwrite its shard for the next call while a slower peer is still copying it
        a.barrier_next(self.SLOT)
        return out


def _wgrad(dy: Tensor, x: Tensor, owners: tuple[Tensor, ...]) -> tuple[Tensor | None, ...]:
    """``dW = dy^T @ x`` for one weight or for several weights that were run as one merged GEMM. Weights that carry
    a ``grad_sink`` (views of a flat data-parallel gradient buffer) receive their gradient there -- one GEMM
    straight into the merged sink when the sinks are adjacent in memory -- and ``None`` is returned for them."""
    from fairseq2_b200.models.transformer.multihead_attention import _merged_sink

    rows = [w.shape[0] for w in owners]
    sink = _merged_sink(owners)
    if sink is not None and sink[0].is_contiguous():
        gemm(dy, x, a_mn=True, b_mn=True, out=sink[0], accumulate=sink[1])
        for w in owners:
            w.grad_sink_filled = True  # type: ignore[attr-defined]
        return tuple(None for _ in owners)
    dw = gemm(dy, x, a_mn=True, b_mn=True)
    return tuple(dw.split(rows, dim=0)) if len(owners) > 1 else (dw,)


class _ColumnSP(torch.autograd.Function):
    """``y [T, F_local] = all_gather(x_shard) @ w^T``; backward reduce-scatters ``dy @ w`` back to the token shard.
    ``w`` may be the merged view of several adjacent weights (``owners``), e.g. q|k|v or gate|up."""

    @staticmethod
    def forward(ctx, x_shard: Tensor, weight: Tensor, sp: "SequenceParallelLinears", *owners: Tensor) -> Tensor:  # type: ignore[override]
        sp.ag.shard.copy_(x_shard)
        y = sp.ag(weight)
        ctx.save_for_backward(x_shard, weight)
        ctx.sp, ctx.owners = sp, owners
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x_shard, weight = ctx.saved_tensors
        sp: SequenceParallelLinears = ctx.sp
        dy = dy.contiguous()
        dx_shard = sp.rs(dy, weight, weight_kn=True) if ctx.needs_input_grad[0] else None   # reduce_scatter(dy @ w)
        owners = ctx.owners
        if owners:
            dws: tuple[Tensor | None, ...] = (None,) * len(owners)
            if any(ctx.needs_input_grad[3:]):
                dws = _wgrad(dy, sp.all_gather_tokens(x_shard), owners)      # [F_local, D] = dy^T @ x
            return (dx_shard, None, None, *dws)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy, sp.all_gather_tokens(x_shard), (weight,))[0]
        return dx_shard, dw, None


class _RowSP(torch.autograd.Function):
    """``y_shard [T / W, D] = reduce_scatter(h @ w^T)``; backward all-gathers ``dy_shard`` inside the dgrad GEMM."""

    @staticmethod
    def forward(ctx, h: Tensor, weight: Tensor, sp: "SequenceParallelLinears") -> Tensor:  # type: ignore[override]
        y = sp.rs(h, weight)
        ctx.save_for_backward(h, weight)
        ctx.sp = sp
        return y

    @staticmethod
    def backward(ctx, dy_shard: Tensor):  # type: ignore[override]
        h, weight = ctx.saved_tensors
        sp: SequenceParallelLinears = ctx.sp
        sp.ag.shard.copy_(dy_shard)
        dh = sp.ag(weight, other_kn=True)                            # [T, F_local] = all_gather(dy) @ w
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _wgrad(sp.ag.gathered, h, (weight,))[0]             # [D, F_local] = dy^T @ h (dy just gathered)
        return dh, dw, None


class SequenceParallelLinears:
    """Megatron-style tensor parallelism with sequence-parallel activations, every collective fused into a GEMM.

    Activations between blocks are sharded by tokens (``[T / W, D]`` per rank). ``column(x_shard, w)`` is the
    column-parallel projection (``w``: ``[F / W, D]``): the all-gather of the tokens runs inside the tcgen05 GEMM.
    ``row(h, w)`` is the row-parallel projection (``w``: ``[D, F / W]``): the GEMM epilogue scatters its tiles to the
    ranks that own the rows and the result comes back token-sharded. The backward passes use the same two kernels
    with the roles swapped, so a feed-forward block costs four fused launches and no stand-alone collective except
    the token all-gather for the column weight gradient. One instance serves all layers of a model with the same
    ``tokens_per_rank`` and ``model_dim`` (the reference has no sequence-parallel mode:
    fairseq2 ``ops/tensor_parallel.py:18-140``, ``nn/projection.py:127-626``).
    """

    def __init__(self, arena: SymmetricArena, tokens_per_rank: int, model_dim: int) -> None:
        self.arena = arena
        self.tokens_per_rank, self.model_dim = tokens_per_rank, model_dim
        self.ag = FusedAllGatherGemm(arena, tokens_per_rank, model_dim, gather="a")
        self.rs = FusedGemmReduceScatter(arena, tokens_per_rank, model_dim, mode="scatter")
        self._gather_off, buf = arena.alloc(tokens_per_rank * model_dim * 2, align=16)
        self._gather_src = buf.view(torch.bfloat16).view(tokens_per_rank, model_dim)
        self._epoch = 0

    def all_gather_tokens(self, x_shard: Tensor) -> Tensor:
        a = self.arena
        self._gather_src.copy_(x_shard)
        n = self.tokens_per_rank * self.model_dim
        full = torch.empty(a.world * n, device=x_shard.device, dtype=torch.bfloat16)
        a.barrier_next(FusedAllGatherGemm.SLOT)                      # every rank has staged its shard
        a.ext.comm_allgather_segments(a.peer_ptrs, a.rank, [0], [n], self._gather_off, full, 1, 0, 8, a.wait_limit_s)
        a.barrier_next(FusedAllGatherGemm.SLOT)                      # nobody restages while a peer still reads
        return full.view(a.world * self.tokens_per_rank, self.model_dim)

    def column(self, x_shard: Tensor, weight: Tensor, owners: tuple[Tensor, ...] = ()) -> Tensor:
        """``owners``: when ``weight`` is a merged view of several adjacent parameters, those parameters (they
        receive the weight gradients)."""
        return _ColumnSP.apply(x_shard, weight, self, *owners)

    def row(self, h: Tensor, weight: Tensor) -> Tensor:
        return _RowSP.apply(h, weight, self)
