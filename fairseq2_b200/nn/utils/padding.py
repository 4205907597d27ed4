"""Stacking variable-length sequences (cf. fairseq2 ``nn/utils/padding.py:17-54``)."""
from __future__ import annotations

from typing import Sequence

import torch
from torch import Tensor

from fairseq2_b200.device import Device
from fairseq2_b200.nn.batch_layout import BatchLayout


def pad_seqs(seqs: Sequence[Tensor], *, pad_value: int = 0, pad_to_multiple: int = 1,
             device: Device | None = None) -> tuple[Tensor, BatchLayout]:
    """Stacks ``seqs`` (equal shapes except dim 0) into ``(N, S, *)``, ``S`` rounded up to ``pad_to_multiple``, and
    returns the stack with its ``BatchLayout``."""
    if len(seqs) == 0:
        raise ValueError("`seqs` must not be empty.")
    if pad_to_multiple < 1:
        raise ValueError(f"`pad_to_multiple` must be at least 1, but is {pad_to_multiple} instead.")
    tail = seqs[0].shape[1:]
    for i, s in enumerate(seqs):
        if s.dim() == 0 or s.shape[1:] != tail:
            raise ValueError(f"All sequences must have the same shape except the first dimension, but `seqs[{i}]` has "
                             f"shape {tuple(s.shape)} and `seqs[0]` {tuple(seqs[0].shape)}.")
    lens = [int(s.shape[0]) for s in seqs]
    width = -(-max(lens) // pad_to_multiple) * pad_to_multiple
    out = seqs[0].new_full((len(seqs), width, *tail), pad_value)
    for i, s in enumerate(seqs):
        out[i, : lens[i]] = s
    if device is not None:
        out = out.to(device, non_blocking=True)
    return out, BatchLayout.of(out, lens)
