"""Synthetic batches of the shapes the benchmark configurations name: packed
SFT sequences made of documents with a masked prompt prefix, and padded
batches. Everything is produced on the host with numpy (as a data pipeline
would) and returned in pinned memory ready for one asynchronous H2D copy."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
from torch import Tensor


@dataclass
class PackedSFTExample:
    tokens: Tensor        # int64 [T + 1]  (inputs = [:-1], targets = [1:])
    target_mask: Tensor   # float32 [T]    (1 where the target token counts)
    seq_lens: list[int]   # document lengths, sum == T
    num_targets: int


def make_packed_sft_example(rng: np.random.Generator, seq_len: int, vocab_size: int,
                            doc_len_range: tuple[int, int] = (128, 4096),
                            prompt_frac_range: tuple[float, float] = (0.1, 0.5), pin: bool = True
                            ) -> PackedSFTExample:
    """Concatenates documents of uniform random length until ``seq_len`` tokens
    are filled (the last one is truncated); per document a uniform-random
    10-50 % prefix is "prompt" whose targets are masked out, and the target
    that would cross into the next document is masked as well."""
    lens: list[int] = []
    total = 0
    while total < seq_len:
        n = int(rng.integers(doc_len_range[0], doc_len_range[1] + 1))
        n = min(n, seq_len - total)
        lens.append(n)
        total += n
    tokens = rng.integers(0, vocab_size, size=seq_len + 1, dtype=np.int64)
    mask = np.ones(seq_len, dtype=np.float32)
    off = 0
    for n in lens:
        frac = rng.uniform(*prompt_frac_range)
        p = int(n * frac)
        # target index i predicts token i + 1; the first p tokens of the document are prompt
        mask[off: off + max(p - 1, 0)] = 0.0
        mask[off + n - 1] = 0.0
        off += n
    t = torch.from_numpy(tokens)
    m = torch.from_numpy(mask)
    if pin and torch.cuda.is_available():
        t, m = t.pin_memory(), m.pin_memory()
    return PackedSFTExample(t, m, lens, int(mask.sum()))
