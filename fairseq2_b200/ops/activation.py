"""SwiGLU gating ``silu(gate) * up``.

The merged gate|up projection writes one ``[T, 2F]`` buffer; the kernel reads
both halves with 16-byte loads and writes ``[T, F]``. Backward recomputes
``silu`` from the saved gate (nothing but the GEMM output is kept alive).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def swiglu_reference(gate_up: Tensor) -> Tensor:
    g, u = gate_up.chunk(2, dim=-1)
    return (F.silu(g.float()) * u.float()).to(gate_up.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up: Tensor) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        gu = gate_up.reshape(-1, gate_up.shape[-1])
        y = ext.swiglu_fwd(gu)
        ctx.save_for_backward(gu)
        return y.view(*gate_up.shape[:-1], gate_up.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        ext = require_ext()
        (gu,) = ctx.saved_tensors
        dgu = ext.swiglu_bwd(dy.reshape(-1, dy.shape[-1]).contiguous(), gu)
        return dgu.view(*dy.shape[:-1], gu.shape[-1])


def swiglu(gate_up: Tensor) -> Tensor:
    """``gate_up[..., :F]`` is the gate, ``gate_up[..., F:]`` the linear branch."""
    if use_kernels(gate_up) and gate_up.dtype == torch.bfloat16 and gate_up.is_contiguous() \
            and gate_up.shape[-1] % 16 == 0:
        return _SwiGLUFn.apply(gate_up)
    return swiglu_reference(gate_up)
