"""Grouped GEMM over row groups (mixture-of-experts feed-forward).

``grouped_mm(x, w, group_sizes)``: ``x`` is ``[T, K]`` with rows sorted by
group, ``w`` is ``[G, K, N]``; rows of group ``g`` are multiplied by ``w[g]``.
On CUDA each group is one tcgen05 GEMM launch writing straight into its row
slice of the output (and, in backward, into its slice of ``dx`` / its page of
``dw``), so nothing is concatenated or copied.
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch import Tensor

from fairseq2_b200.ops.gemm import gemm


def grouped_mm_reference(x: Tensor, w: Tensor, group_sizes: Sequence[int]) -> Tensor:
    out = x.new_empty((x.shape[0], w.shape[2]))
    s = 0
    for g, n in enumerate(group_sizes):
        out[s:s + n] = (x[s:s + n].float() @ w[g].float()).to(x.dtype)
        s += n
    return out


class _GroupedMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, group_sizes: tuple[int, ...]) -> Tensor:  # type: ignore[override]
        x = x.contiguous()
        y = x.new_empty((x.shape[0], w.shape[2]))
        s = 0
        for g, n in enumerate(group_sizes):
            if n:
                gemm(x[s:s + n], w[g], b_mn=True, out=y[s:s + n])
            s += n
        ctx.save_for_backward(x, w)
        ctx.group_sizes = group_sizes
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        dw = torch.zeros_like(w) if ctx.needs_input_grad[1] else None
        s = 0
        for g, n in enumerate(ctx.group_sizes):
            if n:
                if dx is not None:
                    gemm(dy[s:s + n], w[g], out=dx[s:s + n])                    # dy · w[g]ᵀ
                if dw is not None:
                    gemm(x[s:s + n], dy[s:s + n], a_mn=True, b_mn=True, out=dw[g])  # xᵀ · dy
            s += n
        return dx, dw, None


def grouped_mm(x: Tensor, w: Tensor, group_sizes: Sequence[int]) -> Tensor:
    if sum(group_sizes) != x.shape[0]:
        raise ValueError(f"`group_sizes` must sum to the number of rows of `x` ({x.shape[0]}).")
    if len(group_sizes) != w.shape[0]:
        raise ValueError(f"`group_sizes` must have one entry per group of `w` ({w.shape[0]}).")
    return _GroupedMM.apply(x, w, tuple(int(n) for n in group_sizes))


class _GroupedMMDevice(torch.autograd.Function):
    """Single-launch grouped GEMM over the 128-row padded layout; all routing-dependent sizes stay on the device."""

    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, offsets: Tensor, tile_row0: Tensor, tile_expert: Tensor,  # type: ignore[override]
                num_tiles: Tensor) -> Tensor:
        from fairseq2_b200.ops._ext import require_ext

        y = require_ext().grouped_gemm(x.contiguous(), w, True, tile_row0, tile_expert, num_tiles)
        ctx.save_for_backward(x, w, offsets, tile_row0, tile_expert, num_tiles)
        ctx.weight_ref = w if hasattr(w, "grad_sink") else None
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        from fairseq2_b200.ops._ext import require_ext

        ext = require_ext()
        x, w, offsets, tile_row0, tile_expert, num_tiles = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = ext.grouped_gemm(dy, w, False, tile_row0, tile_expert, num_tiles)      # dy @ w[e]^T: w read as [E, K, N] K-major
        if ctx.needs_input_grad[1]:
            dw32 = ext.grouped_gemm_wgrad(x.contiguous(), dy, offsets)                    # [E, K, N] fp32
            wref = ctx.weight_ref
            sink = getattr(wref, "grad_sink", None) if wref is not None else None
            if sink is not None and sink.numel() == dw32.numel():
                # data-parallel wrappers point `grad_sink` into their flat gradient buffer: one conversion pass
                # straight into it instead of a bf16 temporary that is copied again later
                if getattr(wref, "grad_sink_filled", False):
                    sink.view(dw32.shape).add_(dw32)
                else:
                    sink.view(dw32.shape).copy_(dw32)
                wref.grad_sink_filled = True
            else:
                dw = dw32.to(w.dtype)
        return dx, dw, None, None, None, None


def grouped_mm_device_supported(x: Tensor, w: Tensor) -> bool:
    from fairseq2_b200.ops._ext import use_kernels

    return (use_kernels(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 3
            and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0 and w.is_contiguous())


def grouped_mm_device(x: Tensor, w: Tensor, layout: tuple[Tensor, Tensor, Tensor, Tensor]) -> Tensor:
    """``x``: ``[rows, K]`` in the padded expert-sorted layout produced by ``ops.moe.moe_dispatch_padded`` (``layout`` =
    ``(offsets, tile_row0, tile_expert, num_tiles)``), ``w``: ``[E, K, N]`` -> ``[rows, N]``. One kernel launch per
    GEMM, no device-to-host copy of the group sizes."""
    offsets, tile_row0, tile_expert, num_tiles = layout
    return _GroupedMMDevice.apply(x, w, offsets, tile_row0, tile_expert, num_tiles)
