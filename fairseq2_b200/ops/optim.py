"""Multi-tensor AdamW and gradient-norm kernels.

One launch updates a whole list of tensors: fp32 master weights, ``exp_avg``,
``exp_avg_sq`` are read and written once, the gradient (bf16 or fp32) is read
once, and the bf16 compute copy of the parameter is refreshed in the same pass.
The clip coefficient and loss-normalisation factor arrive as *device* scalars
so no host synchronisation sits between backward and the optimizer step.
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def adamw_reference(master: Tensor, grad: Tensor, exp_avg: Tensor, exp_avg_sq: Tensor, *, lr: float, beta1: float,
                    beta2: float, eps: float, weight_decay: float, step: int, grad_scale: Tensor | float = 1.0,
                    low: Tensor | None = None) -> None:
    g = grad.float() * grad_scale
    master.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (exp_avg_sq.sqrt() / (bc2 ** 0.5)).add_(eps)
    master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if low is not None:
        low.copy_(master)


def multi_tensor_adamw(masters: Sequence[Tensor], grads: Sequence[Tensor], exp_avgs: Sequence[Tensor],
                       exp_avg_sqs: Sequence[Tensor], lows: Sequence[Tensor | None], *, lr: float, beta1: float,
                       beta2: float, eps: float, weight_decay: float, step: int,
                       grad_scale: Tensor | None = None) -> None:
    """``grad_scale``: optional fp32 device scalar multiplied into every gradient."""
    if not masters:
        return
    if use_kernels(masters[0]):
        ext = require_ext()
        lows_l = [l if l is not None else torch.empty(0, device=masters[0].device, dtype=torch.bfloat16) for l in lows]
        ext.multi_tensor_adamw(list(masters), list(grads), list(exp_avgs), list(exp_avg_sqs), lows_l,
                               lr, beta1, beta2, eps, weight_decay, step, grad_scale)
        return
    gs: Tensor | float = grad_scale if grad_scale is not None else 1.0
    for p, g, m, v, l in zip(masters, grads, exp_avgs, exp_avg_sqs, lows):
        adamw_reference(p, g, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
                        grad_scale=gs, low=l)


def multi_tensor_l2_norm_sq(tensors: Sequence[Tensor]) -> Tensor:
    """Sum of squares over all tensors as an fp32 device scalar (single pass)."""
    if not tensors:
        return torch.zeros((), dtype=torch.float32)
    if use_kernels(tensors[0]):
        return require_ext().multi_tensor_l2_norm_sq(list(tensors))
    acc = torch.zeros((), dtype=torch.float32, device=tensors[0].device)
    for t in tensors:
        acc += t.float().pow(2).sum()
    return acc


def multi_tensor_scale(tensors: Sequence[Tensor], scale: Tensor | float) -> None:
    if not tensors:
        return
    if use_kernels(tensors[0]) and isinstance(scale, Tensor):
        require_ext().multi_tensor_scale(list(tensors), scale)
        return
    for t in tensors:
        t.mul_(scale)
