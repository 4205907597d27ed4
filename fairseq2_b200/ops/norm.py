"""RMSNorm / LayerNorm (forward and backward).

CUDA: one block per row group, fp32 statistics, 16-byte vector loads, the
backward produces dx in one pass and per-block partial dw that a second tiny
kernel reduces (no atomics, deterministic).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.nn.functional as F
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def rms_norm_reference(x: Tensor, weight: Tensor | None, eps: float, bias: Tensor | None = None) -> Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    y = y.to(x.dtype)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, eps: float) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, rstd = ext.rms_norm_fwd(x2, weight, eps)
        ctx.save_for_backward(x2, weight, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ext = require_ext()
        x2, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx, dw = ext.rms_norm_bwd(dy2, x2, weight, rstd)
        return dx.view(dy.shape), dw.to(weight.dtype), None


class _AddRMSNormFn(torch.autograd.Function):
    """``h = x + res; y = rms_norm(h) * w`` in one kernel; the backward adds the gradient of ``h`` that arrives
    through the residual path to the norm's input gradient in the same pass."""

    @staticmethod
    def forward(ctx, x: Tensor, res: Tensor, weight: Tensor, eps: float):  # type: ignore[override]
        ext = require_ext()
        x2 = x.reshape(-1, x.shape[-1])
        r2 = res.reshape(-1, res.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if not r2.is_contiguous():
            r2 = r2.contiguous()
        h, y, rstd = ext.add_rms_norm_fwd(x2, r2, weight, eps)
        ctx.save_for_backward(h, weight, rstd)
        return h.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, dh: Tensor | None, dy: Tensor | None):  # type: ignore[override]
        ext = require_ext()
        h, weight, rstd = ctx.saved_tensors
        if dy is None:
            return dh, dh, None, None
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dh2 = None
        if dh is not None:
            dh2 = dh.reshape(-1, dh.shape[-1])
            if not dh2.is_contiguous():
                dh2 = dh2.contiguous()
        dx, dw = ext.rms_norm_bwd(dy2, h, weight, rstd, dh2)
        dx = dx.view(dy.shape)
        return dx, dx, dw.to(weight.dtype), None


def add_rms_norm(x: Tensor, res: Tensor, weight: Tensor | None, eps: float) -> tuple[Tensor, Tensor]:
    """Returns ``(x + res, rms_norm(x + res) * weight)``: the residual add and the normalisation that follows it in
    a pre-norm transformer layer, as one pass over the activations on CUDA."""
    if (use_kernels(x) and weight is not None and x.dtype in (torch.bfloat16, torch.float32)
            and weight.dtype == x.dtype and res.dtype == x.dtype and x.shape == res.shape and x.shape[-1] % 8 == 0):
        return _AddRMSNormFn.apply(x, res, weight, eps)
    h = x + res
    return h, rms_norm(h, (h.shape[-1],), weight, eps)


def rms_norm(x: Tensor, normalized_shape: Sequence[int], weight: Tensor | None, eps: float,
             bias: Tensor | None = None) -> Tensor:
    if (use_kernels(x) and weight is not None and bias is None and len(normalized_shape) == 1
            and x.dtype in (torch.bfloat16, torch.float32) and weight.dtype == x.dtype
            and x.shape[-1] % 8 == 0):
        return _RMSNormFn.apply(x, weight, eps)
    if len(normalized_shape) == 1:
        return rms_norm_reference(x, weight, eps, bias)
    dims = tuple(range(-len(normalized_shape), 0))
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(dim=dims, keepdim=True) + eps)).to(x.dtype)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor, eps: float) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, mean, rstd = ext.layer_norm_fwd(x2, weight, bias, eps)
        ctx.save_for_backward(x2, weight, mean, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ext = require_ext()
        x2, weight, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx, dw, db = ext.layer_norm_bwd(dy2, x2, weight, mean, rstd)
        return dx.view(dy.shape), dw.to(weight.dtype), db.to(weight.dtype), None


class _LayerNormGeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor, eps: float) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, mean, rstd = ext.layer_norm_fwd(x2, weight, bias, eps, True)
        ctx.save_for_backward(x2, weight, bias, mean, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ext = require_ext()
        x2, weight, bias, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx, dw, db = ext.layer_norm_bwd(dy2, x2, weight, mean, rstd, bias)
        return dx.view(dy.shape), dw.to(weight.dtype), db.to(weight.dtype), None


def layer_norm_gelu(x: Tensor, weight: Tensor, bias: Tensor, eps: float) -> Tensor:
    """``gelu(layer_norm(x))`` over the last dimension with the exact (erf) GELU, one kernel each way on bf16 CUDA
    tensors: the per-layer tail of a convolutional speech feature encoder on channels-last rows."""
    if (use_kernels(x) and x.dtype == torch.bfloat16 and weight.dtype == x.dtype and bias.dtype == x.dtype
            and x.shape[-1] % 8 == 0):
        return _LayerNormGeluFn.apply(x, weight, bias, eps)
    y = F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps)
    return F.gelu(y).to(x.dtype)


def layer_norm(x: Tensor, normalized_shape: Sequence[int], weight: Tensor | None, bias: Tensor | None,
               eps: float, *, cast_fp32: bool = False) -> Tensor:
    if (use_kernels(x) and weight is not None and bias is not None and len(normalized_shape) == 1
            and x.dtype in (torch.bfloat16, torch.float32) and weight.dtype == x.dtype
            and x.shape[-1] % 8 == 0):
        return _LayerNormFn.apply(x, weight, bias, eps)
    if cast_fp32:
        w = weight.float() if weight is not None else None
        b = bias.float() if bias is not None else None
        return F.layer_norm(x.float(), tuple(normalized_shape), w, b, eps).to(x.dtype)
    return F.layer_norm(x, tuple(normalized_shape), weight, bias, eps)
