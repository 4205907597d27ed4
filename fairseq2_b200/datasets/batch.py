"""Batch containers (cf. fairseq2 ``datasets/batch.py:21-664``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import torch
from torch import Tensor

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.typing import Device


class SequenceBatch:
    """Padded ``(N, S, *)`` or packed ``(T, *)`` sequences with their lengths.

    ``target_mask`` (same leading shape as ``seqs``) marks positions that count
    as targets. ``as_auto_regressive()`` returns ``(input_batch, target_batch)``
    shifted by one position; in packed mode the last position of the buffer is
    trimmed (and the last sequence shortened accordingly).
    """

    def __init__(self, seqs: Tensor, seq_lens: Sequence[int] | None, *, packed: bool = False,
                 target_mask: Tensor | None = None, example: object = None) -> None:
        self.seqs = seqs
        self.packed = packed
        self.target_mask = target_mask
        self.example = example
        if packed:
            if seqs.ndim < 1:
                raise ValueError("`seqs` must be at least one dimensional.")
            self.seq_lens = list(seq_lens) if seq_lens is not None else [seqs.shape[0]]
            if sum(self.seq_lens) > seqs.shape[0]:
                raise ValueError("`sum(seq_lens)` must be less than or equal to the first dimension of `seqs`.")
            self.padding = seqs.shape[0] - sum(self.seq_lens)
        else:
            if seqs.ndim < 2:
                raise ValueError("`seqs` must be at least two dimensional.")
            n, s = seqs.shape[:2]
            self.seq_lens = list(seq_lens) if seq_lens is not None else [s] * n
            if len(self.seq_lens) != n:
                raise ValueError(f"`len(seq_lens)` must equal the batch size ({n}), but is {len(self.seq_lens)}.")
            self.padding = n * s - sum(self.seq_lens)
        if target_mask is not None and target_mask.shape != seqs.shape[: target_mask.ndim]:
            raise ValueError("`target_mask` must have the same leading shape as `seqs`.")
        self._layout: BatchLayout | None = None

    @property
    def batch_size(self) -> int:
        return len(self.seq_lens)

    @property
    def num_examples(self) -> int:
        return len(self.seq_lens)

    @property
    def num_elements(self) -> int:
        return sum(self.seq_lens)

    @property
    def num_target_elements(self) -> int:
        if self.target_mask is None:
            return self.num_elements
        if not hasattr(self, "_num_targets"):
            self._num_targets = int(self.target_mask.sum())
        return self._num_targets

    def as_input(self) -> tuple[Tensor, BatchLayout]:
        if self._layout is None:
            shape = self.seqs.shape[:1] if self.packed else self.seqs.shape[:2]
            self._layout = BatchLayout(tuple(shape), self.seq_lens, packed=self.packed, device=self.seqs.device)
        return self.seqs, self._layout

    def as_auto_regressive(self) -> tuple["SequenceBatch", "SequenceBatch"]:
        if self.packed:
            if self.seqs.shape[0] < 2:
                raise ValueError("The packed batch must hold at least two elements.")
            lens = list(self.seq_lens)
            if self.padding == 0:
                # trim the final element: the last sequence loses one position
                if lens[-1] == 1:
                    lens.pop()
                else:
                    lens[-1] -= 1
            inp, tgt = self.seqs[:-1], self.seqs[1:]
            mask = self.target_mask[1:] if self.target_mask is not None else None
            return (SequenceBatch(inp, lens, packed=True), SequenceBatch(tgt, lens, packed=True, target_mask=mask))
        if self.seqs.shape[1] < 2:
            raise ValueError("The sequence length of `seqs` must be at least 2.")
        lens = [l - 1 for l in self.seq_lens]
        inp, tgt = self.seqs[:, :-1], self.seqs[:, 1:]
        mask = self.target_mask[:, 1:] if self.target_mask is not None else None
        return SequenceBatch(inp, lens), SequenceBatch(tgt, lens, target_mask=mask)

    def to(self, device: Device, *, non_blocking: bool = False) -> "SequenceBatch":
        self.seqs = self.seqs.to(device, non_blocking=non_blocking)
        if self.target_mask is not None:
            self.target_mask = self.target_mask.to(device, non_blocking=non_blocking)
        self._layout = None
        return self

    def pin_memory(self) -> "SequenceBatch":
        self.seqs = self.seqs.pin_memory()
        if self.target_mask is not None:
            self.target_mask = self.target_mask.pin_memory()
        return self


class Seq2SeqBatch:
    def __init__(self, source_seqs: Tensor, source_seq_lens: Sequence[int] | None, target_seqs: Tensor,
                 target_seq_lens: Sequence[int] | None, *, packed: bool = False, target_mask: Tensor | None = None,
                 example: object = None) -> None:
        self.source = SequenceBatch(source_seqs, source_seq_lens, packed=packed)
        self.target = SequenceBatch(target_seqs, target_seq_lens, packed=packed, target_mask=target_mask)
        self.example = example

    @property
    def batch_size(self) -> int:
        return self.target.batch_size

    @property
    def num_examples(self) -> int:
        return self.target.num_examples

    @property
    def num_source_elements(self) -> int:
        return self.source.num_elements

    @property
    def num_target_elements(self) -> int:
        return self.target.num_target_elements

    @property
    def num_elements(self) -> int:
        return self.source.num_elements + self.target.num_elements

    @property
    def padding(self) -> int:
        return self.source.padding + self.target.padding

    def as_source_input(self) -> tuple[Tensor, BatchLayout]:
        return self.source.as_input()

    def as_target_input(self) -> tuple[Tensor, BatchLayout]:
        return self.target.as_input()

    def as_auto_regressive(self) -> tuple["Seq2SeqBatch", SequenceBatch]:
        inp, tgt = self.target.as_auto_regressive()
        b = Seq2SeqBatch.__new__(Seq2SeqBatch)
        b.source, b.target, b.example = self.source, inp, self.example
        return b, tgt

    def to(self, device: Device, *, non_blocking: bool = False) -> "Seq2SeqBatch":
        self.source.to(device, non_blocking=non_blocking)
        self.target.to(device, non_blocking=non_blocking)
        return self
