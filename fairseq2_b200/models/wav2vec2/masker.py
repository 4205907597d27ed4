"""Temporal and spatial span masking (cf. fairseq2 ``models/wav2vec2/masker.py:24-188``)."""
from __future__ import annotations

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.utils.mask import compute_row_mask
from fairseq2_b200.typing import DataType, Device


class Wav2Vec2Masker(Module):
    """Replaces random time spans with a learned embedding and zeroes random feature spans."""

    def __init__(self, model_dim: int, temporal_span_len: int = 10, max_temporal_mask_prob: float = 0.65,
                 min_num_temporal_mask_spans: int = 2, spatial_span_len: int = 10, max_spatial_mask_prob: float = 0.0,
                 min_num_spatial_mask_spans: int = 2, *, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__()
        if max_temporal_mask_prob <= 0.0:
            raise ValueError("`max_temporal_mask_prob` must be greater than 0.")
        self.temporal_span_len, self.max_temporal_mask_prob = temporal_span_len, max_temporal_mask_prob
        self.min_num_temporal_mask_spans = min_num_temporal_mask_spans
        self.temporal_mask_embed = Parameter(torch.empty((model_dim,), device=device, dtype=dtype))
        self.spatial_span_len, self.max_spatial_mask_prob = spatial_span_len, max_spatial_mask_prob
        self.min_num_spatial_mask_spans = min_num_spatial_mask_spans
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.temporal_mask_embed.device.type != "meta":
            torch.nn.init.uniform_(self.temporal_mask_embed)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, Tensor]:
        """Returns the masked sequences and the boolean temporal mask ``(N, S)`` (True = masked)."""
        n, s, m = seqs.shape
        if seqs.is_cuda:
            # The mask is a few thousand booleans whose construction needs several data-dependent sizes (spans per
            # row, masked steps per row). Built on the device, each of them stalls the host until the feature
            # extractor has finished, and the encoder behind it starts with an empty launch queue. The sequence
            # lengths are known on the host, so the mask and the positions it selects are made there and copied.
            host = compute_row_mask((n, s), self.temporal_span_len, self.max_temporal_mask_prob,
                                    row_lens=torch.tensor(list(seqs_layout.seq_lens), dtype=torch.int64),
                                    min_num_spans=self.min_num_temporal_mask_spans, device=torch.device("cpu"))
            if host is None:
                raise ValueError("The temporal mask span length is too long for the given sequences.")
            temporal = host.to(seqs.device, non_blocking=True)
            idx = host.flatten().nonzero().squeeze(1)
            temporal._fs2_masked_rows = idx.to(seqs.device, non_blocking=True)  # type: ignore[attr-defined]
        else:
            temporal = compute_row_mask((n, s), self.temporal_span_len, self.max_temporal_mask_prob,
                                        row_lens=seqs_layout.seq_lens_pt,
                                        min_num_spans=self.min_num_temporal_mask_spans, device=seqs.device)
            if temporal is None:
                raise ValueError("The temporal mask span length is too long for the given sequences.")
        seqs = torch.where(temporal.unsqueeze(-1), self.temporal_mask_embed.to(seqs.dtype), seqs)
        if self.max_spatial_mask_prob > 0.0:
            spatial = compute_row_mask((n, m), self.spatial_span_len, self.max_spatial_mask_prob,
                                       min_num_spans=self.min_num_spatial_mask_spans, device=seqs.device)
            if spatial is None:
                raise ValueError("The spatial mask span length is too long for the model dimension.")
            seqs = seqs.masked_fill(spatial.unsqueeze(1), 0.0)
        return seqs, temporal

    @staticmethod
    def extract_masked_elements(seqs: Tensor, temporal_mask: Tensor) -> Tensor:
        """``(N, S, M)`` -> ``(N, S_masked, M)``; every row of the mask selects the same number of steps."""
        n = seqs.shape[0]
        rows = getattr(temporal_mask, "_fs2_masked_rows", None)
        if rows is not None and rows.device == seqs.device:
            # positions computed on the host together with the mask: a gather, no `nonzero` round trip
            return seqs.flatten(0, 1).index_select(0, rows).unflatten(0, (n, -1))
        return seqs[temporal_mask].unflatten(0, (n, -1))

    def extra_repr(self) -> str:
        return (f"temporal_span_len={self.temporal_span_len}, max_temporal_mask_prob={self.max_temporal_mask_prob}, "
                f"spatial_span_len={self.spatial_span_len}, max_spatial_mask_prob={self.max_spatial_mask_prob}")
