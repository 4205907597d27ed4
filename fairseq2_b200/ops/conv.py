"""Strided 1-D convolution over channels-last signals as a tcgen05 GEMM on overlapping-row views.

For ``x`` ``[B, L, C]`` (contiguous) and a kernel of width ``k`` and stride ``s`` with ``L % s == 0``, row ``r`` of the
patch matrix is ``x.flatten()[r * s * C : r * s * C + k * C]`` -- consecutive rows overlap in memory. A TMA tensor map
with row pitch ``s * C`` describes exactly that matrix, so the convolution is ONE GEMM ``patches @ W2^T`` with
``W2 = weight.permute(0, 2, 1).reshape(C_out, k * C)`` and no im2col buffer. The backward uses the same views:

* weight gradient ``dW2 = dY^T @ patches`` (both operands MN-major views),
* input gradient: ``dY @ W2`` has the shape of the patch matrix; the GEMM epilogue reduce-adds it through the same
  overlapping-row tensor map into a zeroed ``dx``, which sums the overlapping taps (col2im without a buffer).

The output has ``L / s`` rows per batch element ("virtual length"): row ``t`` is a true convolution output iff
``t * s + k <= valid_len``; the remaining rows at the end of each batch element mix in the next element's samples (or
zeros at the very end) and must be dropped by the caller -- stacks of such layers drop them once at the end, since a
valid row of layer ``i + 1`` only ever reads valid rows of layer ``i``.

Replaces cuDNN ``Conv1d`` + two transposes per layer in the wav2vec2 feature extractor
(fairseq2 ``models/wav2vec2/feature_extractor.py:28-270``) for the layers with 8-element-aligned channel counts.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def conv1d_cl_reference(x: Tensor, weight: Tensor, bias: Tensor | None, stride: int) -> Tensor:
    """fp32 oracle with the same virtual-length convention (invalid tail rows are zero-padded convolutions)."""
    B, L, C = x.shape
    k = weight.shape[2]
    xp = F.pad(x.float().transpose(1, 2), (0, k))                 # tail rows read zeros here, neighbours in the kernel
    y = F.conv1d(xp, weight.float(), None if bias is None else bias.float(), stride=stride)
    return y[:, :, : L // stride].transpose(1, 2)


def conv1d_cl_supported(x: Tensor, weight: Tensor, stride: int) -> bool:
    C_out, C, k = weight.shape
    return (use_kernels(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 3
            and x.shape[2] == C and C % 8 == 0 and C_out % 8 == 0 and x.shape[1] % stride == 0 and k >= stride
            and x.shape[0] * x.shape[1] * C >= k * C)


class _Conv1dCL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, stride: int) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        B, L, C = x.shape
        C_out, _, k = weight.shape
        x = x.contiguous()
        w2 = weight.permute(0, 2, 1).reshape(C_out, k * C).contiguous()
        R = B * L // stride                                       # rows of the (virtual) patch matrix
        rows_ok = (B * L * C - k * C) // (stride * C) + 1         # rows that lie fully inside the storage
        y = torch.empty((R, C_out), device=x.device, dtype=x.dtype)
        ext.gemm_bf16_view(x, min(rows_ok, R), stride * C, False, w2, C_out, k * C, False, y, R, C_out, R, C_out, k * C,
                           False, 1)
        ctx.save_for_backward(x, w2)
        ctx.meta = (B, L, C, C_out, k, stride, R, min(rows_ok, R))
        return y.view(B, L // stride, C_out)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ext = require_ext()
        x, w2 = ctx.saved_tensors
        B, L, C, C_out, k, stride, R, rows_ok = ctx.meta
        dy2 = dy.reshape(R, C_out).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[1]:
            # dW2 [C_out, k*C] = dY^T [C_out, R] @ patches [R, k*C]; rows of the patch view beyond rows_ok read zeros
            # a long reduction (all output positions) into a small matrix: split K so that every SM has a tile
            tiles = ((C_out + 127) // 128) * ((k * C + 255) // 256)
            splits = max(1, min(R // 2048, (2 * 148 + tiles - 1) // tiles))
            dw2 = torch.zeros((C_out, k * C), device=x.device, dtype=torch.float32)
            ext.gemm_bf16_view(dy2, R, C_out, True, x, rows_ok, stride * C, True, dw2, C_out, k * C, C_out, k * C, R,
                               True, splits)
            dw = dw2.view(C_out, k, C).permute(0, 2, 1).to(w2.dtype)
        if ctx.needs_input_grad[0]:
            # d patches [R, k*C] = dY [R, C_out] @ W2 [C_out, k*C], reduce-added through the overlapping-row view
            # overlapping taps add at most ceil(k / stride) bf16 partial sums per element
            dx2 = torch.zeros((B * L, C), device=x.device, dtype=x.dtype)
            ext.gemm_bf16_view(dy2, R, C_out, False, w2, C_out, k * C, True, dx2, rows_ok, stride * C, R, k * C, C_out,
                               True, 1)
            dx = dx2.view(B, L, C)
        return dx, dw, None


def conv1d_channels_last(x: Tensor, weight: Tensor, bias: Tensor | None, stride: int) -> Tensor:
    """``x`` ``[B, L, C_in]``, ``weight`` ``[C_out, C_in, k]`` (the ``torch.nn.Conv1d`` layout) -> ``[B, L / stride,
    C_out]`` in the virtual-length convention of the module docstring."""
    if conv1d_cl_supported(x, weight, stride):
        y = _Conv1dCL.apply(x, weight, stride)
        return y if bias is None else y + bias
    return conv1d_cl_reference(x, weight, bias, stride).to(x.dtype)


# ---------------------------------------------------------------- first feature-extractor layer
def first_conv_reference(x: Tensor, weight: Tensor, bias: Tensor | None, ln_weight: Tensor | None,
                         ln_bias: Tensor | None, stride: int, t_pad: int, eps: float) -> Tensor:
    """fp32 formulation of :func:`first_conv_ln_gelu` (any device): ``[B, L]`` -> ``[B, t_pad, C]``."""
    y = F.conv1d(x.float().unsqueeze(1), weight.float(), None if bias is None else bias.float(), stride=stride)
    y = y.transpose(1, 2)
    if ln_weight is not None:
        y = F.gelu(F.layer_norm(y, (y.shape[-1],), ln_weight.float(), None if ln_bias is None else ln_bias.float(), eps))
    return F.pad(y, (0, 0, 0, t_pad - y.shape[1]))


class _FirstConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, ln_weight, ln_bias, stride, t_pad, eps):  # type: ignore[no-untyped-def]
        ext = require_ext()
        w2 = weight.reshape(weight.shape[0], weight.shape[2]).contiguous()
        ctx.save_for_backward(x, w2, bias, ln_weight, ln_bias)
        ctx.meta = (stride, eps, weight.shape)
        return ext.w2v_first_conv_fwd(x, w2, bias, ln_weight, ln_bias, stride, t_pad, eps)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[no-untyped-def]
        x, w2, bias, ln_weight, ln_bias = ctx.saved_tensors
        stride, eps, wshape = ctx.meta
        dw, db, dlw, dlb = require_ext().w2v_first_conv_bwd(dy.contiguous(), x, w2, bias, ln_weight, ln_bias, stride, eps)
        return (None, dw.view(wshape).to(w2.dtype), None if bias is None else db.to(bias.dtype),
                None if ln_weight is None else dlw.to(ln_weight.dtype),
                None if ln_bias is None else dlb.to(ln_bias.dtype), None, None, None)


def first_conv_supported(x: Tensor, weight: Tensor) -> bool:
    return (use_kernels(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and weight.dim() == 3 and weight.shape[1] == 1 and not x.requires_grad
            and require_ext().w2v_first_conv_supported(weight.shape[0], weight.shape[2])
            and x.shape[1] >= weight.shape[2])


def first_conv_ln_gelu(x: Tensor, weight: Tensor, bias: Tensor | None, ln_weight: Tensor | None,
                       ln_bias: Tensor | None, stride: int, t_pad: int | None = None, eps: float = 1e-5) -> Tensor:
    """First layer of the wav2vec 2.0 feature extractor in one kernel: ``x`` ``[B, L]`` waveform, ``weight``
    ``[C, 1, k]`` -> channels-last ``[B, t_pad, C]`` = ``GELU(LayerNorm(conv1d(x) + bias))`` (the bare convolution
    + bias when ``ln_weight`` is ``None``); rows past the ``(L - k) // stride + 1`` true outputs are zero. The layer
    is bound by writing its output, so the convolution, the normalisation over the channels and the activation run
    in registers between one read of the waveform and one write of the result; the backward recomputes the row from
    the waveform (nothing but the inputs is saved) and produces the four parameter gradients. Replaces cuDNN
    ``Conv1d`` + transpose + LayerNorm + GELU + transpose + pad
    (fairseq2 ``models/wav2vec2/feature_extractor.py:129-172``)."""
    t_valid = (x.shape[1] - weight.shape[2]) // stride + 1
    if t_pad is None:
        t_pad = t_valid
    if first_conv_supported(x, weight):
        return _FirstConv.apply(x.contiguous(), weight, bias, ln_weight, ln_bias, stride, t_pad, eps)
    return first_conv_reference(x, weight, bias, ln_weight, ln_bias, stride, t_pad, eps).to(x.dtype)


# ------------------------------------------------------------------------ grouped convolution
def grouped_conv1d_supported(x: Tensor, weight: Tensor, groups: int) -> bool:
    C_out, Cg, k = weight.shape
    return (use_kernels(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 3
            and groups > 1 and x.shape[2] == Cg * groups and C_out % groups == 0 and Cg % 8 == 0
            and (C_out // groups) % 8 == 0)


def grouped_conv1d_channels_last(x: Tensor, weight: Tensor, bias: Tensor | None, groups: int, padding: int) -> Tensor:
    """Stride-1 grouped convolution over a channels-last signal: ``x`` ``[B, T, C]``, ``weight``
    ``[C_out, C / groups, k]`` (the ``torch.nn.Conv1d`` layout), zero padding on both sides ->
    ``[B, T + 2 * padding - k + 1, C_out]``.

    The signal is copied once into a group-major, zero-padded layout ``[groups, B, T_p, C / groups]``; there the
    patch matrix of a group is an overlapping-row view (row pitch ``C / groups``, row length ``k * C / groups``) and
    the group's convolution is one tcgen05 GEMM of :func:`conv1d_channels_last`, as are its two gradients. For the
    positional convolution of wav2vec 2.0 (k = 128, 16 groups of 64 channels) that is a ``[B * T_p, 8192] x [8192,
    64]`` GEMM per group instead of cuDNN's grouped implicit-GEMM kernels
    (fairseq2 ``models/wav2vec2/position_encoder.py:69-107``)."""
    B, T, C = x.shape
    C_out, Cg, k = weight.shape
    if not grouped_conv1d_supported(x, weight, groups):
        y = F.conv1d(x.transpose(1, 2), weight, bias, padding=padding, groups=groups)
        return y.transpose(1, 2)
    Og = C_out // groups
    Tp = T + 2 * padding
    xg = F.pad(x, (0, 0, padding, padding)).view(B, Tp, groups, Cg).permute(2, 0, 1, 3).contiguous()
    outs = [conv1d_channels_last(xg[g], weight[g * Og:(g + 1) * Og], None, 1) for g in range(groups)]
    y = torch.stack(outs, dim=2)[:, : Tp - k + 1].reshape(B, Tp - k + 1, C_out)      # rows past that are not outputs
    return y if bias is None else y + bias
