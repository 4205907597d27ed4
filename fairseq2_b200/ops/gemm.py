"""Dense bf16 GEMM on tcgen05/TMEM.

``gemm(a, b, a_mn=, b_mn=)`` computes ``C[M, N] = A · Bᵀ`` where, with the
default *K-major* operands, ``a`` is ``[M, K]`` and ``b`` is ``[N, K]`` (the
``F.linear`` convention). An *MN-major* operand is stored transposed: ``a`` as
``[K, M]`` (``a_mn=True``), ``b`` as ``[K, N]`` (``b_mn=True``). This covers the
three GEMMs of a linear layer without materialising any transpose:

* forward ``y = x Wᵀ``            -> ``gemm(x, W)``
* dgrad   ``dx = dy W``           -> ``gemm(dy, W, b_mn=True)``
* wgrad   ``dW = dyᵀ x``          -> ``gemm(dy, x, a_mn=True, b_mn=True)``

The kernel is a persistent, warp-specialised TMA -> smem -> ``tcgen05.mma`` ->
TMEM pipeline (see ``csrc/gemm_tcgen05.cu``). Shapes with at least half a wave
of 256 x 256 tiles run on pairs of CTAs (``cta_group::2``: one tile per two
SMs, each CTA stages half of ``b``); ``FAIRSEQ2_B200_GEMM_PAIR=0`` keeps them
on the single-CTA kernel. When the last wave of tiles is partial, its tiles are
cut into two K slices that are reduce-added (deterministic: a + b in either
order), so a bf16 result can differ from the single-pass one by one rounding.
"""
from __future__ import annotations

import os

import torch
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def gemm_reference(a: Tensor, b: Tensor, *, a_mn: bool = False, b_mn: bool = False,
                   out_dtype: torch.dtype | None = None) -> Tensor:
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    return (A.float() @ B.float()).to(out_dtype or a.dtype)


def _kernel_ok(a: Tensor, b: Tensor) -> bool:
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        return False
    if a.ndim != 2 or b.ndim != 2 or not a.is_contiguous() or not b.is_contiguous():
        return False
    # TMA: 16-byte aligned base and row pitch.
    if a.shape[1] % 8 or b.shape[1] % 8 or a.data_ptr() % 16 or b.data_ptr() % 16:
        return False
    return True


_USE_CUBLAS = os.environ.get("FAIRSEQ2_B200_GEMM", "tcgen05") == "cublas"


def gemm(a: Tensor, b: Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Tensor | None = None,
         out_dtype: torch.dtype | None = None, accumulate: bool = False) -> Tensor:
    """See module docstring. ``accumulate=True`` adds into ``out`` (fp32 or bf16)."""
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    if K != Kb:
        raise ValueError(f"The reduction dimensions of `a` ({K}) and `b` ({Kb}) do not match.")
    if use_kernels(a, b) and not _USE_CUBLAS and _kernel_ok(a, b):
        odt = out.dtype if out is not None else (out_dtype or torch.bfloat16)
        if out is None:
            out = torch.empty((M, N), dtype=odt, device=a.device)
            accumulate = False
        if out.is_contiguous() and out.shape == (M, N) and N % 8 == 0 and odt in (torch.bfloat16, torch.float32) \
                and M > 0 and N > 0 and K > 0:
            require_ext().gemm_bf16(a, b, out, a_mn, b_mn, accumulate)
            return out
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    if out is None:
        r = torch.matmul(A, B)
        return r if out_dtype is None or out_dtype == r.dtype else r.to(out_dtype)
    if accumulate:
        out.add_(torch.matmul(A, B).to(out.dtype))
    else:
        out.copy_(torch.matmul(A, B))
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor) -> Tensor:  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = x.shape
        ctx.weight_ref = weight if hasattr(weight, "grad_sink") else None
        y = gemm(x2, weight)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            w = ctx.weight_ref
            sink = getattr(w, "grad_sink", None) if w is not None else None
            if sink is not None and sink.is_contiguous():
                # data-parallel wrappers point `grad_sink` into their flat gradient buffer
                gemm(dy2, x2, a_mn=True, b_mn=True, out=sink, accumulate=bool(getattr(w, "grad_sink_filled", False)))
                w.grad_sink_filled = True
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """``x Wᵀ (+ b)``; CUDA bf16 inputs run on the tcgen05 GEMM with its own backward."""
    if use_kernels(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and not _USE_CUBLAS \
            and weight.is_contiguous() and weight.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0:
        y = _LinearFn.apply(x, weight)
        if bias is not None:
            y = y + bias
        return y
    return torch.nn.functional.linear(x, weight, bias)


class _LinearKNFn(torch.autograd.Function):
    """``y = x @ w`` with ``w`` stored ``[K, N]`` (an MN-major B operand): no transpose is ever materialised."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, out_dtype: torch.dtype | None = None) -> Tensor:  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = x.shape
        return gemm(x2, weight, b_mn=True, out_dtype=out_dtype).view(*x.shape[:-1], weight.shape[1])

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(x2.dtype)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, weight).view(ctx.x_shape) if ctx.needs_input_grad[0] else None     # dy [M, N] x w [K, N]^T
        dw = gemm(x2, dy2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None     # x^T dy -> [K, N]
        return dx, dw, None


def linear_kn(x: Tensor, weight: Tensor, out_dtype: torch.dtype | None = None) -> Tensor:
    """``x @ weight`` for a weight stored ``[in, out]`` (e.g. a mixture-of-experts router); CUDA bf16 inputs run on
    the tcgen05 GEMM, forward and backward. ``out_dtype=torch.float32`` keeps the fp32 accumulators (router logits
    decide a discrete choice, so they are not rounded to bf16)."""
    if use_kernels(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and not _USE_CUBLAS \
            and weight.is_contiguous() and weight.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0:
        return _LinearKNFn.apply(x, weight, out_dtype)
    y = x @ weight
    return y.to(out_dtype) if out_dtype is not None else y
