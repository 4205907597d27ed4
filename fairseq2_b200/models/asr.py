"""Speech recognition model interface (cf. fairseq2 ``models/asr.py:19-80``)."""
from __future__ import annotations

from abc import ABC, abstractmethod

from torch import Tensor
from torch.nn import Module

from fairseq2_b200.nn.batch_layout import BatchLayout


class AsrModel(Module, ABC):
    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, targets: Tensor | None = None,
                targets_layout: BatchLayout | None = None, *, return_logits: bool = False
                ) -> Tensor | tuple[Tensor, BatchLayout] | tuple[Tensor, Tensor, BatchLayout]:
        """Without ``targets``: ``(logits, layout)``. With ``targets``: the CTC loss, or
        ``(loss, logits, layout)`` when ``return_logits``."""
