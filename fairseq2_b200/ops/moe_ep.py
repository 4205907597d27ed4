"""Expert-parallel token exchange for mixture-of-experts layers, fused into the routing kernels.

Rank r of an expert-parallel group of W ranks owns experts ``[r * E / W, (r + 1) * E / W)``. The two all-to-alls of
the usual formulation (tokens to experts, expert outputs back to tokens) do not exist as separate collectives here:

* **dispatch** -- after a one-block kernel has exchanged the per-expert counts (every rank learns the layout of every
  inbox), one kernel stores each selected token row, scaled by its gate if asked, straight into the inbox of the rank
  that owns the expert (16-byte stores over NVLink). Inbox rows are grouped by local expert, ready for the grouped GEMM.
* **combine** -- one kernel loads, for each local token, its ``k`` expert outputs straight from the owners' outboxes
  (16-byte peer loads) and sums them, weighted by the gates if asked.

Both are differentiable: the backward of dispatch is a combine over the gradient of the inbox rows (which also yields
the gate gradients as dot products), the backward of combine is a dispatch of the output gradient to the same rows.
Buffers live in a ``SymmetricArena``; ordering between ranks uses its epoch-flag barriers (bounded waits).

The reference keeps MoE experts tensor-parallel only and lets every expert process every token (fairseq2
``models/llama4/moe.py:109-157``); this operator is what its inline comment calls for and has no reference counterpart.
"""

from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.parallel.symm import SymmetricArena


def ep_reference(x_all: list[Tensor], ids_all: list[Tensor], gates_all: list[Tensor], expert_fn, rank: int,
                 scale_input: bool) -> Tensor:  # type: ignore[no-untyped-def]
    """Dense fp32 oracle for ``rank``'s tokens: ``y[t] = sum_j w_out * expert_{id}(w_in * x[t])``."""
    x, ids, gates = x_all[rank].float(), ids_all[rank].long(), gates_all[rank].float()
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(ids.shape[1]):
            g = gates[t, j]
            inp = x[t] * g if scale_input else x[t]
            out = expert_fn(int(ids[t, j]), inp.to(torch.bfloat16).float())
            y[t] += out if scale_input else g * out
    return y


class _Push(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ep: "ExpertParallelExchange", x: Tensor, gates: Tensor | None, expert_ids: Tensor,  # type: ignore[override]
                counts: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        a = ep.arena
        send_base, cursor, group_sizes, total = a.ext.moe_ep_layout(a.peer_ptrs, a.rank, counts, ep.table_off, ep.SLOT,
                                                                    ep.next_epoch(), a.wait_limit_s)
        dest = torch.empty_like(expert_ids)
        a.ext.moe_ep_push(a.peer_ptrs, a.rank, x, expert_ids, gates, send_base, cursor, ep.inbox_off, dest,
                          ep.num_experts, ep.capacity)
        a.barrier(ep.SLOT, ep.next_epoch())                     # every rank's rows have landed in my inbox
        sizes = group_sizes.tolist()
        n = sum(sizes)
        if n > ep.capacity:
            raise RuntimeError(f"The expert inbox holds {ep.capacity} rows but {n} were routed to this rank.")
        rows = ep.inbox[:n].clone()                              # the inbox is reused by the next exchange
        ctx.ep, ctx.has_gates = ep, gates is not None
        ctx.save_for_backward(x, gates if gates is not None else x.new_empty(0), dest)
        ctx.mark_non_differentiable(dest, group_sizes)
        return rows, dest, group_sizes

    @staticmethod
    def backward(ctx, d_rows: Tensor, *_: Tensor):  # type: ignore[override]
        ep: ExpertParallelExchange = ctx.ep
        a = ep.arena
        x, gates, dest = ctx.saved_tensors
        n = d_rows.shape[0]
        ep.outbox[:n].copy_(d_rows)
        a.barrier(ep.SLOT, ep.next_epoch())                     # every owner has published its row gradients
        dx = torch.empty_like(x)
        if ctx.has_gates:
            dgates = torch.empty(dest.shape, device=x.device, dtype=torch.float32)
            a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, gates, dx, x, dgates, ep.capacity, False)
        else:
            dgates = None
            a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, None, dx, None, None, ep.capacity, False)
        a.barrier(ep.SLOT, ep.next_epoch())                     # outboxes may be overwritten again
        return None, dx, dgates, None, None


class _Pull(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ep: "ExpertParallelExchange", rows: Tensor, dest: Tensor, gates: Tensor | None,  # type: ignore[override]
                base: Tensor | None, num_tokens: int) -> Tensor:
        a = ep.arena
        n = rows.shape[0]
        ep.outbox[:n].copy_(rows)
        a.barrier(ep.SLOT, ep.next_epoch())                     # every owner has published its expert outputs
        y = base.clone() if base is not None else torch.empty((num_tokens, rows.shape[1]), device=rows.device,
                                                              dtype=rows.dtype)
        a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, gates, y, None, None, ep.capacity, base is not None)
        a.barrier(ep.SLOT, ep.next_epoch())                     # outboxes may be overwritten again
        ctx.ep, ctx.n, ctx.has_gates, ctx.has_base = ep, n, gates is not None, base is not None
        ctx.save_for_backward(dest, gates if gates is not None else rows.new_empty(0), rows)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ep: ExpertParallelExchange = ctx.ep
        a = ep.arena
        dest, gates, rows = ctx.saved_tensors
        dy = dy.contiguous()
        dgates = None
        if ctx.has_gates:
            # d gate[t, j] = <expert output row, dy[t]>: pull the rows once more, dotted with dy
            ep.outbox[: ctx.n].copy_(rows)
            a.barrier(ep.SLOT, ep.next_epoch())
            dgates = torch.empty(dest.shape, device=dy.device, dtype=torch.float32)
            scratch = torch.empty_like(dy)
            a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, None, scratch, dy, dgates, ep.capacity, False)
            a.barrier(ep.SLOT, ep.next_epoch())
        # d rows: the output gradient travels to the rows the tokens were sent to
        a.ext.moe_ep_push(a.peer_ptrs, a.rank, dy, None, gates if ctx.has_gates else None, None, None, ep.inbox_off,
                          dest, ep.num_experts, ep.capacity)
        a.barrier(ep.SLOT, ep.next_epoch())
        d_rows = ep.inbox[: ctx.n].clone()
        return None, d_rows, None, dgates, (dy if ctx.has_base else None), None


class _PushPadded(torch.autograd.Function):
    """Dispatch into the 128-row padded inbox layout of the single-launch grouped GEMM. Nothing returns to the host:
    the received rows are handed on as a capacity-sized buffer together with device-resident tile tables."""

    @staticmethod
    def forward(ctx, ep: "ExpertParallelExchange", x: Tensor, gates: Tensor | None, expert_ids: Tensor,  # type: ignore[override]
                counts: Tensor):
        a = ep.arena
        (send_base, limit, cursor, offsets, group_sizes, tile_row0, tile_expert, num_tiles, total) = \
            a.ext.moe_ep_layout_padded(a.peer_ptrs, a.rank, counts, ep.table_off, ep.inbox_off, ep.capacity,
                                       ep.model_dim, ep.SLOT, ep.next_epoch(), a.wait_limit_s)
        dest = torch.empty_like(expert_ids)
        a.ext.moe_ep_push(a.peer_ptrs, a.rank, x, expert_ids, gates, send_base, cursor, ep.inbox_off, dest,
                          ep.num_experts, ep.capacity, limit, ep.dropped)
        a.barrier(ep.SLOT, ep.next_epoch())                     # every rank's rows have landed in my inbox
        rows = torch.empty_like(ep.inbox)                        # the inbox is reused by the next exchange
        a.ext.copy_rows_bounded(rows, ep.inbox, num_tiles)       # (only the rows that hold data are copied)
        ctx.ep, ctx.has_gates = ep, gates is not None
        ctx.save_for_backward(x, gates if gates is not None else x.new_empty(0), dest, num_tiles)
        ctx.mark_non_differentiable(dest, offsets, group_sizes, tile_row0, tile_expert, num_tiles, total)
        return rows, dest, offsets, group_sizes, tile_row0, tile_expert, num_tiles, total

    @staticmethod
    def backward(ctx, d_rows: Tensor, *_: Tensor):  # type: ignore[override]
        ep: ExpertParallelExchange = ctx.ep
        a = ep.arena
        x, gates, dest, num_tiles = ctx.saved_tensors
        a.ext.copy_rows_bounded(ep.outbox, d_rows.contiguous(), num_tiles)
        a.barrier(ep.SLOT, ep.next_epoch())                     # every owner has published its row gradients
        dx = torch.empty_like(x)
        if ctx.has_gates:
            dgates = torch.empty(dest.shape, device=x.device, dtype=torch.float32)
            a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, gates, dx, x, dgates, ep.capacity, False)
        else:
            dgates = None
            a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, None, dx, None, None, ep.capacity, False)
        a.barrier(ep.SLOT, ep.next_epoch())                     # outboxes may be overwritten again
        return None, dx, dgates, None, None


class _PullPadded(torch.autograd.Function):
    """Combine from capacity-sized outboxes (the counterpart of ``_PushPadded``)."""

    @staticmethod
    def forward(ctx, ep: "ExpertParallelExchange", rows: Tensor, dest: Tensor, gates: Tensor | None,  # type: ignore[override]
                base: Tensor | None, num_tokens: int, num_tiles: Tensor | None = None) -> Tensor:
        a = ep.arena
        a.ext.copy_rows_bounded(ep.outbox, rows, num_tiles)
        a.barrier(ep.SLOT, ep.next_epoch())                     # every owner has published its expert outputs
        y = base.clone() if base is not None else torch.empty((num_tokens, rows.shape[1]), device=rows.device,
                                                              dtype=rows.dtype)
        a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, gates, y, None, None, ep.capacity, base is not None)
        a.barrier(ep.SLOT, ep.next_epoch())                     # outboxes may be overwritten again
        ctx.ep, ctx.has_gates, ctx.has_base, ctx.bounded = ep, gates is not None, base is not None, num_tiles is not None
        ctx.save_for_backward(dest, gates if gates is not None else rows.new_empty(0),
                              rows if gates is not None else rows.new_empty(0),
                              num_tiles if num_tiles is not None else dest.new_empty(0))
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ep: ExpertParallelExchange = ctx.ep
        a = ep.arena
        dest, gates, rows, num_tiles = ctx.saved_tensors
        nt = num_tiles if ctx.bounded else None
        dy = dy.contiguous()
        dgates = None
        if ctx.has_gates:
            a.ext.copy_rows_bounded(ep.outbox, rows, nt)
            a.barrier(ep.SLOT, ep.next_epoch())
            dgates = torch.empty(dest.shape, device=dy.device, dtype=torch.float32)
            scratch = torch.empty_like(dy)
            a.ext.moe_ep_pull(a.peer_ptrs, a.rank, ep.outbox_off, dest, None, scratch, dy, dgates, ep.capacity, False)
            a.barrier(ep.SLOT, ep.next_epoch())
        # d rows: the output gradient travels to the rows the tokens were sent to (dropped rows go nowhere)
        a.ext.moe_ep_push(a.peer_ptrs, a.rank, dy, None, gates if ctx.has_gates else None, None, None, ep.inbox_off,
                          dest, ep.num_experts, ep.capacity)
        a.barrier(ep.SLOT, ep.next_epoch())
        # The row gradients are consumed straight from the inbox: the experts' backward runs before this rank
        # reaches the barriers of the dispatch's backward, and no peer can start the exchange that next writes
        # this inbox before it has passed those barriers.
        return None, ep.inbox, None, dgates, (dy if ctx.has_base else None), None, None


class ExpertParallelExchange:
    """Buffers and epoch bookkeeping of one expert-parallel group; shared by all MoE layers of a model.

    ``capacity`` is the number of rows an inbox can hold; the default ``world * max_tokens * top_k`` can never
    overflow. Every rank must call ``dispatch`` / ``combine`` (and run backward) the same number of times.
    """

    SLOT = 44

    def __init__(self, arena: SymmetricArena, num_experts: int, model_dim: int, max_tokens: int, top_k: int,
                 capacity: int | None = None) -> None:
        W = arena.world
        if num_experts % W:
            raise ValueError(f"`num_experts` ({num_experts}) must be a multiple of the group size ({W}).")
        if model_dim % 8:
            raise ValueError("`model_dim` must be a multiple of 8.")
        self.arena, self.num_experts, self.model_dim = arena, num_experts, model_dim
        self.num_local_experts = num_experts // W
        cap = capacity if capacity is not None else W * max_tokens * top_k
        # whole 128-row tiles, and room for the padding of the tile-aligned per-expert ranges
        self.capacity = max((cap + 127) // 128 * 128 + 128 * self.num_local_experts, 128 * self.num_local_experts)
        #: rows that did not fit into an inbox since creation (device counter; 0 unless ``capacity`` was set too low)
        self.dropped = torch.zeros(1, dtype=torch.int32, device=arena.device)
        self.table_off, _ = arena.alloc(4 * W * num_experts, align=16)
        self.inbox_off, inbox = arena.alloc(self.capacity * model_dim * 2, align=16)
        self.outbox_off, outbox = arena.alloc(self.capacity * model_dim * 2, align=16)
        self.inbox = inbox.view(torch.bfloat16).view(self.capacity, model_dim)
        self.outbox = outbox.view(torch.bfloat16).view(self.capacity, model_dim)
        self._epoch = 0
        arena.barrier(self.SLOT, self.next_epoch())

    def next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch

    def dispatch(self, x: Tensor, expert_ids: Tensor, counts: Tensor, gates: Tensor | None = None
                 ) -> tuple[Tensor, Tensor, Tensor]:
        """``x`` [T, D] bf16, ``expert_ids`` [T, k] int32 (global expert ids), ``counts`` [E] int32.

        Returns ``(rows, dest, group_sizes)``: the rows this rank's experts must process, grouped by local expert
        (``group_sizes`` [E / W]), and the handle ``dest`` that ``combine`` needs. With ``gates`` the rows are
        ``x[t] * gate[t, j]``."""
        g = gates.float().contiguous() if gates is not None else None
        return _Push.apply(self, x.contiguous(), g, expert_ids.contiguous(), counts.contiguous())

    def combine(self, rows: Tensor, dest: Tensor, num_tokens: int, gates: Tensor | None = None,
                base: Tensor | None = None, num_tiles: Tensor | None = None) -> Tensor:
        """``y[t] = base[t] + sum_j gate[t, j] * rows_of_owner[dest[t, j]]`` (gate = 1 if not given). ``num_tiles``
        (from the layout of :meth:`dispatch_padded`): only that many 128-row tiles of ``rows`` hold data."""
        g = gates.float().contiguous() if gates is not None else None
        if rows.shape[0] == self.capacity:
            return _PullPadded.apply(self, rows.contiguous(), dest, g, base, num_tokens, num_tiles)
        return _Pull.apply(self, rows.contiguous(), dest, g, base, num_tokens)

    def dispatch_padded(self, x: Tensor, expert_ids: Tensor, counts: Tensor, gates: Tensor | None = None
                        ) -> tuple[Tensor, Tensor, tuple[Tensor, Tensor, Tensor, Tensor], Tensor]:
        """Like :meth:`dispatch`, but the received rows come as the whole ``[capacity, D]`` inbox in the 128-row
        padded layout of the single-launch grouped GEMM, with its device-resident tables: returns
        ``(rows, dest, (offsets, tile_row0, tile_expert, num_tiles), group_sizes)``. The host never waits for the
        routing result. Rows that do not fit into an inbox are dropped and counted in ``self.dropped``."""
        g = gates.float().contiguous() if gates is not None else None
        rows, dest, offsets, group_sizes, tile_row0, tile_expert, num_tiles, _ = _PushPadded.apply(
            self, x.contiguous(), g, expert_ids.contiguous(), counts.contiguous())
        return rows, dest, (offsets, tile_row0, tile_expert, num_tiles), group_sizes
