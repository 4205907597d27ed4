"""Rotary position encoding on interleaved pairs.

``x[..., 2i], x[..., 2i+1]`` is rotated by the angle ``pos * theta_i``. The
kernel rotates q and k heads in place right after the QKV projection, reading
positions (``-1`` = padding -> left untouched/zero angle) from the batch layout
and a precomputed fp32 ``[max_len, D/2, 2]`` (cos, sin) table. Backward is the
same kernel with the angle negated.
"""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def rope_reference(x: Tensor, freqs: Tensor, positions: Tensor, inverse: bool = False) -> Tensor:
    """``x``: ``[*, S, H, D]`` or ``[*, S, D]``; ``freqs``: ``[L, D/2, 2]`` (cos, sin);
    ``positions``: integer ``[*, S]`` with -1 at padding."""
    has_heads = x.ndim == positions.ndim + 2
    f = freqs[(positions.clamp(min=0)).long()]  # [*, S, D/2, 2]
    if has_heads:
        f = f.unsqueeze(-3)
    cos, sin = f[..., 0], f[..., 1]
    if inverse:
        sin = -sin
    xf = x.float().unflatten(-1, (-1, 2))
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
    return out.to(x.dtype)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, freqs: Tensor, positions: Tensor) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        ctx.save_for_backward(freqs, positions)
        y = x.contiguous().clone() if x.requires_grad or not x.is_contiguous() else x.clone()
        ext.rope_inplace(y.view(-1, y.shape[-2], y.shape[-1]), freqs, positions.reshape(-1), False)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ext = require_ext()
        freqs, positions = ctx.saved_tensors
        dx = dy.contiguous().clone()
        ext.rope_inplace(dx.view(-1, dx.shape[-2], dx.shape[-1]), freqs, positions.reshape(-1), True)
        return dx, None, None


def apply_rope(x: Tensor, freqs: Tensor, positions: Tensor) -> Tensor:
    """``x``: ``[..., S, H, D]``; ``positions``: int32 ``[..., S]``."""
    if use_kernels(x) and x.dtype == torch.bfloat16 and positions.dtype == torch.int32 \
            and x.ndim == positions.ndim + 2 and x.shape[-1] % 8 == 0:
        return _RopeFn.apply(x, freqs, positions)
    return rope_reference(x, freqs, positions)
