"""Loss functions (cf. fairseq2 ``nn/functional/cross_entropy.py:16-185``)."""
from __future__ import annotations

from typing import Literal

from torch import Tensor

from fairseq2_b200.ops.cross_entropy import cross_entropy_reference, fused_linear_cross_entropy  # noqa: F401


def cross_entropy(logits: Tensor, targets: Tensor, pad_idx: int | None, *, label_smoothing: float = 0.0,
                  target_mask: Tensor | None = None,
                  reduction: Literal["sum", "mean", "none"] = "sum") -> Tensor:
    """fp32 log-softmax cross entropy with ``pad_idx`` ignore and optional
    ``target_mask``; label smoothing is fairseq-compatible."""
    batch = logits.shape[0] if logits.ndim == 3 else None
    loss = cross_entropy_reference(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), pad_idx,
                                   target_mask=target_mask.reshape(-1) if target_mask is not None else None,
                                   label_smoothing=label_smoothing, reduction=reduction)
    if reduction == "none" and batch is not None:
        loss = loss.view(batch, -1)
    return loss
