"""Gradient utilities (cf. fairseq2 ``nn/utils/grad.py:25-159``).

``normalize_grads`` turns the data-parallel *mean* of per-rank sum-losses into
the gradient of the global mean loss: scale by ``dp.size / total_targets``.
In this framework the scale factor stays on the device so the hot loop never
synchronises; data-parallel wrappers that own flat gradient buffers consume the
factor inside their fused optimizer step instead of a separate pass.
"""
from __future__ import annotations

from typing import Iterable

import torch
from torch import Tensor
from torch.nn import Module

from fairseq2_b200.error import InternalError
from fairseq2_b200.gang import Gang, ReduceOperation, all_sum
from fairseq2_b200.ops.optim import multi_tensor_l2_norm_sq, multi_tensor_scale


def _grads(module: Module) -> list[Tensor]:
    return [p.grad for p in module.parameters() if p.grad is not None]


def scale_grads(module: Module, value: float | Tensor) -> None:
    gs = _grads(module)
    if not gs:
        return
    if isinstance(value, Tensor) and gs[0].is_cuda:
        multi_tensor_scale(gs, value.to(device=gs[0].device, dtype=torch.float32))
    else:
        for g in gs:
            g.mul_(value)


def normalize_grads(module: Module, gang: Gang, num_targets: int | Tensor, *, foreach: bool = False) -> Tensor:
    """Scales gradients by ``gang.size / sum_over_ranks(num_targets)``; returns the factor."""
    total = all_sum(gang, num_targets)
    factor = gang.size / total.to(torch.float32)
    scale_grads(module, factor)
    return factor


def _tensor_parallel_split(module: Module) -> tuple[Gang | None, set[int]]:
    """The tensor-parallel gang of ``module`` (``None`` if it has none) and the ids of the parameters that are
    split over it."""
    from fairseq2_b200.nn.sharded import Sharded

    gang: Gang | None = None
    split: set[int] = set()
    for m in module.modules():
        if isinstance(m, Sharded):
            g = getattr(m, "gang", None)
            if g is not None and g.size > 1:
                gang = g
                split.update(id(p) for p, _ in m.get_shard_dims())
    return gang, split


def clip_grad_norm(module: Module, max_norm: float | None, norm_type: float = 2.0) -> Tensor:
    """Global gradient norm; clips in place when ``max_norm`` is given. In a tensor-parallel model the norm covers
    the whole model: the squared norms of the parameters that are split over the gang are summed over it, those of
    the replicated parameters count once, so every rank scales by the same factor."""
    gs = _grads(module)
    if not gs:
        return torch.zeros(())
    tp, split = _tensor_parallel_split(module)
    if tp is not None:
        if norm_type != 2.0:
            raise ValueError("Only the 2-norm is supported for tensor-parallel models.")
        dev = gs[0].device
        parts = torch.zeros(2, device=dev, dtype=torch.float32)        # [split over the gang, replicated]
        for p in module.parameters():
            if p.grad is not None:
                parts[0 if id(p) in split else 1] += p.grad.detach().float().pow(2).sum()
        shared = parts[:1].clone()
        tp.all_reduce(shared, ReduceOperation.SUM)
        total = (shared[0] + parts[1]).sqrt()
        if max_norm is not None:
            coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
            for g in gs:
                g.mul_(coef.to(g.dtype))
        return total
    if norm_type == 2.0 and gs[0].is_cuda and all(g.is_contiguous() and g.data_ptr() % 16 == 0 for g in gs):
        total = multi_tensor_l2_norm_sq(gs).sqrt()
        if max_norm is not None:
            coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
            multi_tensor_scale(gs, coef)
        return total
    return torch.nn.utils.clip_grad_norm_(module.parameters(), max_norm if max_norm is not None else torch.inf,
                                          norm_type)


def check_grad_norms(local_norm: Tensor, gang: Gang, step_nr: int) -> bool:
    """True when every rank reports the same (finite) gradient norm."""
    if gang.size == 1:
        return True
    norms = torch.zeros((gang.size,), device=gang.device, dtype=local_norm.dtype)
    gang.all_gather(norms.view(gang.size, *local_norm.shape) if local_norm.ndim else norms.view(gang.size),
                    local_norm.detach().to(gang.device))
    if not torch.isfinite(norms).all():
        return False
    ref = norms[0]
    return bool(((norms - ref).abs() <= 1e-5 * ref.abs().clamp(min=1.0)).all())
