"""Span masking (cf. fairseq2 ``nn/utils/mask.py:18-205``): ``compute_row_mask``
draws, per row, random spans of ``span_len`` covering ~``max_mask_prob`` of the
row, as used by wav2vec2 time/feature masking."""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.typing import Device


def apply_mask(seqs: Tensor, mask: Tensor, fill_value: int | float | Tensor = 0) -> Tensor:
    """Elements where ``mask`` is False are replaced by ``fill_value``."""
    if mask.ndim < seqs.ndim:
        mask = mask.view(*mask.shape, *([1] * (seqs.ndim - mask.ndim)))
    return seqs.where(mask, fill_value) if not isinstance(fill_value, Tensor) else torch.where(mask, seqs, fill_value)


def compute_row_mask(shape: tuple[int, int], span_len: int, max_mask_prob: float, row_lens: Tensor | None = None,
                     min_num_spans: int = 0, device: Device | None = None, generator: torch.Generator | None = None
                     ) -> Tensor | None:
    """Boolean ``shape`` mask; True marks masked positions. Returns ``None`` if
    no row is long enough to hold a span."""
    num_rows, max_row_len = shape
    if row_lens is None:
        if span_len >= max_row_len:
            raise ValueError(f"The size of the second dimension of `shape` must be greater than `span_len` ({span_len}), but is {max_row_len} instead.")
        row_lens = torch.full((num_rows,), max_row_len, device=device, dtype=torch.int64)
    else:
        row_lens = row_lens.view(num_rows).to(device=device, dtype=torch.int64)
        if (span_len >= row_lens).any():
            raise ValueError(f"All lengths in `row_lens` must be greater than `span_len` ({span_len}).")
    dev = row_lens.device
    # number of spans per row: prob * len / span_len plus a random rounding term
    rnd = torch.rand(num_rows, device=dev, generator=generator)
    num_spans = ((max_mask_prob / span_len) * (row_lens - 1) + rnd).to(torch.int64)
    if min_num_spans > 0:
        num_spans = num_spans.clamp(min=min_num_spans)
    # the same number of spans for every row keeps the op batched (as the reference does): use the minimum
    n = int(num_spans.min())
    if n == 0:
        return None
    span_start_range = (row_lens - span_len + 1).view(num_rows, 1)
    starts = (torch.rand((num_rows, n), device=dev, generator=generator) * span_start_range).to(torch.int64)
    offs = torch.arange(span_len, device=dev).view(1, 1, span_len)
    idx = (starts.unsqueeze(-1) + offs).view(num_rows, -1)
    mask = torch.zeros((num_rows, max_row_len), device=dev, dtype=torch.bool)
    mask.scatter_(1, idx.clamp(max=max_row_len - 1), True)
    valid = torch.arange(max_row_len, device=dev).view(1, -1) < row_lens.view(-1, 1)
    mask &= valid
    # Overlapping spans leave rows with different numbers of masked elements. Consumers gather the masked
    # elements into a dense (rows, count) tensor, so surplus elements are unmasked at random: every masked
    # element draws a key and only the `min count` smallest keys of a row stay masked.
    counts = mask.sum(dim=1)
    keep = int(counts.min())
    if keep < int(counts.max()):
        keys = torch.rand(mask.shape, device=dev, generator=generator).masked_fill_(~mask, 2.0)
        kth = keys.kthvalue(keep, dim=1, keepdim=True).values if keep > 0 else keys.new_full((num_rows, 1), -1.0)
        mask &= keys <= kth
    return mask
