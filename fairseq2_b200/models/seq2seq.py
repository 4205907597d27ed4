"""Sequence-to-sequence model interface (cf. fairseq2 ``models/seq2seq.py:19-126``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Literal

from torch import Tensor
from torch.nn import Module

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag


class Seq2SeqModel(Module, ABC):
    def __init__(self, max_source_seq_len: int, max_target_seq_len: int) -> None:
        super().__init__()
        self.max_source_seq_len, self.max_target_seq_len = max_source_seq_len, max_target_seq_len

    @abstractmethod
    def forward(self, source_seqs: Tensor, source_seqs_layout: BatchLayout, target_seqs: Tensor,
                target_seqs_layout: BatchLayout, targets: Tensor | None = None, *,
                state_bag: IncrementalStateBag | None = None, label_smoothing: float = 0.0,
                target_mask: Tensor | None = None, reduction: Literal["sum", "mean"] = "sum",
                return_logits: bool = False) -> Tensor | tuple[Tensor, Tensor]:
        """Without ``targets``: logits. With ``targets``: the loss, or ``(loss, logits)``."""
