"""Causal language model interface (cf. fairseq2 ``models/clm.py:18``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Literal

from torch import Tensor
from torch.nn import Module

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag


class CausalLM(Module, ABC):
    def __init__(self, max_seq_len: int) -> None:
        super().__init__()
        self.max_seq_len = max_seq_len

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, targets: Tensor | None = None, *,
                state_bag: IncrementalStateBag | None = None, label_smoothing: float = 0.0,
                target_mask: Tensor | None = None, reduction: Literal["sum", "mean"] = "sum",
                return_logits: bool = False) -> Tensor | tuple[Tensor, Tensor]:
        """Without ``targets``: logits. With ``targets``: the loss, or
        ``(loss, logits)`` when ``return_logits``."""
