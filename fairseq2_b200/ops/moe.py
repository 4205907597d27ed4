"""Mixture-of-experts routing on the GPU: fused top-k gate + expert histogram, dispatch (gather + gate scaling
into expert-sorted order) and combine (gather back per token), each a single sm_100a kernel with its own
backward. The PyTorch formulations are the CPU path and the oracles."""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def moe_route_reference(logits: Tensor, k: int, softmax_gate: bool = False) -> tuple[Tensor, Tensor, Tensor]:
    """``(expert_ids [T, k], gates [T, k], counts [E])``."""
    top, ids = torch.topk(logits.float(), k, dim=1)
    gates = torch.softmax(top, dim=1) if softmax_gate else torch.sigmoid(top)
    counts = torch.bincount(ids.reshape(-1), minlength=logits.shape[1])
    return ids, gates, counts


class _Dispatch(torch.autograd.Function):
    """``routed[slot] = x[t] * gate[t, j]`` for ``slot = inv[t, j]``."""

    @staticmethod
    def forward(ctx, x: Tensor, gates: Tensor, expert_ids: Tensor, counts: Tensor):  # type: ignore[override]
        ext = require_ext()
        routed, src_row, inv, offsets = ext.moe_dispatch(x, expert_ids, gates, counts, True)
        ctx.save_for_backward(x, gates, src_row, inv)
        ctx.mark_non_differentiable(src_row, inv, offsets)
        return routed, src_row, inv, offsets

    @staticmethod
    def backward(ctx, d_routed: Tensor, *_: Tensor):  # type: ignore[override]
        ext = require_ext()
        x, gates, src_row, inv = ctx.saved_tensors
        d_routed = d_routed.contiguous()
        dx = torch.empty_like(x)
        ext.moe_combine(d_routed, inv, gates, dx, False)                     # dx[t] = sum_j g[t,j] * d_routed[slot]
        # d gate[t, j] = <d_routed[slot], x[t]>
        xr = x.index_select(0, src_row.long())
        dslot = (d_routed.float() * xr.float()).sum(dim=1)
        dgates = dslot[inv.long()]
        return dx, dgates, None, None


class _DispatchPadded(torch.autograd.Function):
    """``_Dispatch`` into the 128-row padded layout of the single-launch grouped GEMM (padding rows are zero)."""

    @staticmethod
    def forward(ctx, x: Tensor, gates: Tensor, expert_ids: Tensor, counts: Tensor):  # type: ignore[override]
        ext = require_ext()
        routed, src_row, inv, offsets, tile_row0, tile_expert, num_tiles = ext.moe_dispatch_padded(
            x, expert_ids, gates, counts, True)
        ctx.save_for_backward(x, gates, src_row, inv)
        ctx.mark_non_differentiable(src_row, inv, offsets, tile_row0, tile_expert, num_tiles)
        return routed, src_row, inv, offsets, tile_row0, tile_expert, num_tiles

    @staticmethod
    def backward(ctx, d_routed: Tensor, *_: Tensor):  # type: ignore[override]
        ext = require_ext()
        x, gates, src_row, inv = ctx.saved_tensors
        d_routed = d_routed.contiguous()
        dx = torch.empty_like(x)
        ext.moe_combine(d_routed, inv, gates, dx, False)
        live = src_row >= 0
        xr = x.index_select(0, src_row.clamp(min=0).long())
        dslot = (d_routed.float() * xr.float()).sum(dim=1) * live
        dgates = dslot[inv.long()]
        return dx, dgates, None, None


class _Combine(torch.autograd.Function):
    """``y[t] = base[t] + sum_j routed[inv[t, j]]``."""

    @staticmethod
    def forward(ctx, routed: Tensor, inv: Tensor, src_row: Tensor, base: Tensor | None):  # type: ignore[override]
        ext = require_ext()
        T = inv.shape[0]
        y = base.clone() if base is not None else torch.empty((T, routed.shape[1]), device=routed.device,
                                                              dtype=routed.dtype)
        ext.moe_combine(routed.contiguous(), inv, None, y, base is not None)
        ctx.save_for_backward(inv, src_row)
        ctx.has_base = base is not None
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        inv, src_row = ctx.saved_tensors
        dy = dy.contiguous()
        d_routed = dy.index_select(0, src_row.clamp(min=0).long())
        if bool((src_row.numel() > 0)):
            d_routed = d_routed * (src_row >= 0).unsqueeze(1).to(d_routed.dtype)    # padding rows of the padded layout
        return d_routed, None, None, (dy if ctx.has_base else None)


def moe_kernels_available(x: Tensor, logits: Tensor) -> bool:
    return (use_kernels(x, logits) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and logits.shape[-1] <= 256)


def moe_route(logits: Tensor, k: int, softmax_gate: bool = False) -> tuple[Tensor, Tensor, Tensor]:
    """Top-k routing. On CUDA the gates are differentiable with respect to ``logits`` through a cheap PyTorch
    re-evaluation of the selected logits (the selection itself comes from the fused kernel)."""
    if use_kernels(logits) and logits.dtype in (torch.bfloat16, torch.float32) and logits.shape[1] <= 256 and k <= 8:
        ids, _, counts, _ = require_ext().moe_route(logits.detach().contiguous(), k, softmax_gate, False)
        sel = logits.float().gather(1, ids.long())
        gates = torch.softmax(sel, dim=1) if softmax_gate else torch.sigmoid(sel)
        return ids, gates, counts
    ids, gates, counts = moe_route_reference(logits, k, softmax_gate)
    return ids.to(torch.int32), gates, counts.to(torch.int32)


def moe_dispatch(x: Tensor, gates: Tensor, expert_ids: Tensor, counts: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    """Returns ``(routed [T·k, D] in expert order, src_row [T·k], inv [T, k])``."""
    routed, src_row, inv, _ = _Dispatch.apply(x.contiguous(), gates.float().contiguous(), expert_ids.contiguous(),
                                              counts.contiguous())
    return routed, src_row, inv


def moe_dispatch_padded(x: Tensor, gates: Tensor, expert_ids: Tensor, counts: Tensor
                        ) -> tuple[Tensor, Tensor, Tensor, tuple[Tensor, Tensor, Tensor, Tensor]]:
    """Like ``moe_dispatch`` but into a buffer whose per-expert row ranges are padded to multiples of 128 rows, with
    the tile tables the single-launch grouped GEMM needs. Returns ``(routed, src_row, inv, layout)``; nothing is
    copied to the host."""
    routed, src_row, inv, offsets, tile_row0, tile_expert, num_tiles = _DispatchPadded.apply(
        x.contiguous(), gates.float().contiguous(), expert_ids.contiguous(), counts.contiguous())
    return routed, src_row, inv, (offsets, tile_row0, tile_expert, num_tiles)


def moe_combine(routed: Tensor, inv: Tensor, src_row: Tensor, base: Tensor | None = None) -> Tensor:
    return _Combine.apply(routed, inv, src_row, base)


def load_balancing_loss(logits: Tensor, counts: Tensor, top_k: int) -> Tensor:
    """Switch / GShard load-balancing auxiliary loss of one router:
    ``E * sum_e f_e * P_e`` with ``f_e`` the fraction of the ``T * k`` routing slots that went to expert ``e`` (a
    constant with respect to the parameters) and ``P_e`` the mean router probability of expert ``e``. It is 1 for a
    uniform router and grows as load and probability mass concentrate on the same experts. ``logits``: ``[T, E]``;
    ``counts``: ``[E]`` slots per expert as produced by the routing kernel."""
    T, E = logits.shape
    probs = torch.softmax(logits.float(), dim=-1).mean(dim=0)
    frac = counts.to(torch.float32) / max(T * top_k, 1)
    return E * (frac.detach() * probs).sum()


class _SwiGLU2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g: Tensor, u: Tensor, num_tiles: Tensor | None) -> Tensor:  # type: ignore[override]
        g, u = g.contiguous(), u.contiguous()
        ctx.save_for_backward(g, u, num_tiles if num_tiles is not None else g.new_empty(0))
        ctx.bounded = num_tiles is not None
        return require_ext().swiglu2_fwd(g, u, num_tiles)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        g, u, nt = ctx.saved_tensors
        dg, du = require_ext().swiglu2_bwd(dy.contiguous(), g, u, nt if ctx.bounded else None)
        return dg, du, None


def swiglu_gate_up(g: Tensor, u: Tensor, num_tiles: Tensor | None = None) -> Tensor:
    """``silu(g) * u`` for the separate gate / up outputs of the grouped expert GEMMs in one pass (and one pass
    backward). ``num_tiles`` (device int32): only the first ``num_tiles * 128`` rows of the capacity-sized buffers
    hold data; the rest is neither read nor written."""
    if use_kernels(g, u) and g.dtype == torch.bfloat16 and g.dim() == 2 and g.shape[1] % 8 == 0:
        return _SwiGLU2.apply(g, u, num_tiles)
    return torch.nn.functional.silu(g) * u
