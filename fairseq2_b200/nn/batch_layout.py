"""Layout descriptor of padded ``(N, S)`` and packed ``(T,)`` batches.

API parity with fairseq2 ``nn/batch_layout.py:20-233``. The B200-first
difference is how device metadata is produced: all index vectors are computed
on the host with numpy into ONE pinned int32 staging buffer and shipped with a
single asynchronous H2D copy; the device views (``seq_begin_indices_pt``,
``seq_lens_pt``, ``position_indices``) are slices of that one allocation.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch
from torch import Tensor

from fairseq2_b200.typing import Device


class BatchLayout:
    def __init__(self, shape: tuple[int, ...], seq_lens: Sequence[int] | None, *, packed: bool = False,
                 device: Device | None = None) -> None:
        self._packed = packed
        if packed:
            if len(shape) != 1:
                raise ValueError(f"`shape` must be 1 dimensional, but is {len(shape)} dimensional instead.")
            width = int(shape[0])
            if width < 1:
                raise ValueError("`shape[0]` must be greater than or equal to 1.")
            lens = np.asarray([width] if seq_lens is None else list(seq_lens), dtype=np.int64)
            self._check_lens(lens)
            total = int(lens.sum())
            if total > width:
                raise ValueError(
                    f"`sum(seq_lens)` must be less than or equal to `shape[0]` ({width}), but is {total} instead.")
            begins = np.zeros(len(lens) + 1, dtype=np.int64)
            np.cumsum(lens, out=begins[1:])
            pos = np.full(width, -1, dtype=np.int64)
            if total:
                pos[:total] = np.arange(total) - np.repeat(begins[:-1], lens)
            self._padded = total < width
            pos_shape: tuple[int, ...] = (width,)
        else:
            if len(shape) != 2:
                raise ValueError(f"`shape` must be 2 dimensional, but is {len(shape)} dimensional instead.")
            n, width = int(shape[0]), int(shape[1])
            if width < 1:
                raise ValueError("`shape[1]` must be greater than or equal to 1.")
            lens = np.asarray([width] * n if seq_lens is None else list(seq_lens), dtype=np.int64)
            if len(lens) != n:
                raise ValueError(f"`len(seq_lens)` must be equal to `shape[0]` ({n}), but is {len(lens)} instead.")
            self._check_lens(lens)
            if n and int(lens.max()) > width:
                idx = int(np.argmax(lens > width))
                raise ValueError(
                    f"All lengths in `seq_lens` must be less than or equal to `shape[1]` ({width}), but the length at index {idx} is {int(lens[idx])} instead.")
            begins = np.arange(0, n * width + 1, width, dtype=np.int64)
            ar = np.arange(width, dtype=np.int64)
            pos = np.where(ar[None, :] < lens[:, None], ar[None, :], -1)
            self._padded = bool(n and int(lens.min()) < width)
            pos_shape = (n, width)

        self._width = width
        self._seq_lens = lens.tolist()
        self._seq_begin_indices = begins.tolist()
        self._min_seq_len = int(lens.min()) if len(lens) else width
        self._max_seq_len = int(lens.max()) if len(lens) else 0

        nb, nl, npos = len(begins), len(lens), pos.size
        dev = device or torch.device("cpu")
        if dev.type == "cuda":
            stage = torch.empty(nb + nl + npos, dtype=torch.int32, pin_memory=True)
            buf = stage.numpy()
            buf[:nb], buf[nb:nb + nl], buf[nb + nl:] = begins, lens, pos.reshape(-1)
            meta = stage.to(dev, non_blocking=True)
            self._stage = stage  # keeps the pinned block alive until the copy ran
        else:
            meta = torch.from_numpy(np.concatenate([begins, lens, pos.reshape(-1)]).astype(np.int32)).to(dev)
        self._seq_begin_indices_pt = meta[:nb]
        self._seq_lens_pt = meta[nb:nb + nl]
        self._position_indices_i32 = meta[nb + nl:].view(pos_shape)
        self._position_indices: Tensor | None = None

    @staticmethod
    def _check_lens(lens: np.ndarray) -> None:
        if len(lens) and int(lens.min()) < 1:
            idx = int(np.argmax(lens < 1))
            raise ValueError(
                f"All lengths in `seq_lens` must be greater than or equal to 1, but the length at index {idx} is {int(lens[idx])} instead.")

    @staticmethod
    def of(batch: Tensor, seq_lens: Sequence[int] | None = None, *, packed: bool = False) -> "BatchLayout":
        shape = batch.shape[:1] if packed else batch.shape[:2]
        return BatchLayout(tuple(shape), seq_lens, packed=packed, device=batch.device)

    @property
    def width(self) -> int:
        return self._width

    @property
    def seq_begin_indices(self) -> Sequence[int]:
        return self._seq_begin_indices

    @property
    def seq_begin_indices_pt(self) -> Tensor:
        """int32 ``[num_seqs + 1]`` (the ``cu_seqlens`` of varlen attention)."""
        return self._seq_begin_indices_pt

    @property
    def seq_lens(self) -> Sequence[int]:
        return self._seq_lens

    @property
    def seq_lens_pt(self) -> Tensor:
        return self._seq_lens_pt

    @property
    def min_seq_len(self) -> int:
        return self._min_seq_len

    @property
    def max_seq_len(self) -> int:
        return self._max_seq_len

    @property
    def position_indices(self) -> Tensor:
        """int64 positions within each sequence, -1 at padding."""
        if self._position_indices is None:
            self._position_indices = self._position_indices_i32.long()
        return self._position_indices

    @property
    def position_indices_i32(self) -> Tensor:
        """The same positions as int32 (what the fused RoPE kernels consume)."""
        return self._position_indices_i32

    @property
    def padded(self) -> bool:
        return self._padded

    @property
    def packed(self) -> bool:
        return self._packed

    def __repr__(self) -> str:
        return (f"BatchLayout(width={self._width}, seq_begin_indices={self._seq_begin_indices}, "
                f"seq_lens={self._seq_lens}, min_seq_len={self._min_seq_len}, max_seq_len={self._max_seq_len}, "
                f"padded={self._padded}, packed={self._packed})")
