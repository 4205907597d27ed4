"""Autograd-aware tensor-parallel collectives (cf. fairseq2 ``ops/tensor_parallel.py:20-134``).

``reduce``: all-reduce fwd / identity bwd. ``reduce_on_backward``: identity fwd
/ all-reduce bwd. ``scatter``: keep own slice fwd / all-gather bwd. ``gather``:
all-gather fwd / slice bwd. Additionally the sequence-parallel pair
``reduce_scatter_seq`` / ``all_gather_seq`` used by the fused TP linears.
"""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.gang import Gang, ReduceOperation


def _all_gather_dim(x: Tensor, gang: Gang, dim: int) -> Tensor:
    if gang.size == 1:
        return x
    out = x.new_empty((gang.size, *x.shape))
    gang.all_gather(out, x.contiguous())
    dim = dim % x.ndim
    return torch.cat(list(out.unbind(0)), dim=dim) if dim != 0 else out.flatten(0, 1)


def _slice_dim(x: Tensor, gang: Gang, dim: int) -> Tensor:
    if gang.size == 1:
        return x
    n = x.shape[dim]
    if n % gang.size:
        raise ValueError(f"The size of dimension {dim} ({n}) must be a multiple of the gang size ({gang.size}).")
    c = n // gang.size
    return x.narrow(dim, gang.rank * c, c).contiguous()


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gang: Gang) -> Tensor:  # type: ignore[override]
        y = x.detach().clone()
        gang.all_reduce(y, ReduceOperation.SUM)
        return y

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return g, None


class _ReduceOnBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gang: Gang) -> Tensor:  # type: ignore[override]
        ctx.gang = gang
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        g = g.contiguous().clone()
        ctx.gang.all_reduce(g, ReduceOperation.SUM)
        return g, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gang: Gang, dim: int) -> Tensor:  # type: ignore[override]
        ctx.gang, ctx.dim = gang, dim
        return _slice_dim(x, gang, dim)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return _all_gather_dim(g, ctx.gang, ctx.dim), None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gang: Gang, dim: int) -> Tensor:  # type: ignore[override]
        ctx.gang, ctx.dim = gang, dim
        return _all_gather_dim(x, gang, dim)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return _slice_dim(g, ctx.gang, ctx.dim), None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gang: Gang, dim: int) -> Tensor:  # type: ignore[override]
        ctx.gang, ctx.dim = gang, dim
        n = gang.size
        xs = torch.stack(x.chunk(n, dim=dim), dim=0).contiguous()
        out = torch.empty_like(xs[0])
        gang.reduce_scatter(out, xs, ReduceOperation.SUM)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return _all_gather_dim(g, ctx.gang, ctx.dim), None, None


class _ReduceBothWays(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gang: Gang) -> Tensor:  # type: ignore[override]
        ctx.gang = gang
        y = x.clone()
        gang.all_reduce(y, ReduceOperation.SUM)
        return y

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        g = g.clone()
        ctx.gang.all_reduce(g, ReduceOperation.SUM)
        return g, None


def reduce_both_ways(x: Tensor, gang: Gang) -> Tensor:
    """Sum over the gang in the forward AND the backward pass: for a value that every rank computes a part of and
    then uses in its own shard of a computation (a statistic over a dimension that is split over the ranks), so that
    both the parts and the gradients of the uses add up."""
    if gang.size == 1:
        return x
    return _ReduceBothWays.apply(x, gang)


def reduce(x: Tensor, gang: Gang) -> Tensor:
    return x if gang.size == 1 else _Reduce.apply(x, gang)


def reduce_on_backward(x: Tensor, gang: Gang) -> Tensor:
    return x if gang.size == 1 else _ReduceOnBackward.apply(x, gang)


def scatter(x: Tensor, gang: Gang, dim: int = -1) -> Tensor:
    return x if gang.size == 1 else _Scatter.apply(x, gang, dim)


def gather(x: Tensor, gang: Gang, dim: int = -1) -> Tensor:
    return x if gang.size == 1 else _Gather.apply(x, gang, dim)


def reduce_scatter_seq(x: Tensor, gang: Gang, dim: int = 0) -> Tensor:
    """Sum over the gang and keep this rank's slice of ``dim`` (bwd: all-gather)."""
    return x if gang.size == 1 else _ReduceScatter.apply(x, gang, dim)


def all_gather_seq(x: Tensor, gang: Gang, dim: int = 0) -> Tensor:
    """All-gather along ``dim`` whose backward is a reduce-scatter."""
    if gang.size == 1:
        return x

    class _AG(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t: Tensor) -> Tensor:  # type: ignore[override]
            return _all_gather_dim(t, gang, dim)

        @staticmethod
        def backward(ctx, g: Tensor):  # type: ignore[override]
            n = gang.size
            gs = torch.stack(g.chunk(n, dim=dim), dim=0).contiguous()
            out = torch.empty_like(gs[0])
            gang.reduce_scatter(out, gs, ReduceOperation.SUM)
            return out

    return _AG.apply(x)
