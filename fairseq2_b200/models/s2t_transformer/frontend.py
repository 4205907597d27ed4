"""Speech-to-text front end (cf. fairseq2 ``models/s2t_transformer/feature_extractor.py:23-133``,
``models/s2t_transformer/frontend.py:27-103``): two stride-2 GLU convolutions subsample the filter-bank
frames by four, then scale, add positions, optionally project (Conformer) and drop out."""
from __future__ import annotations

import math
from typing import Sequence

from torch import Tensor
from torch.nn import GLU, Conv1d, Dropout, Module, Sequential

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.models.feature_extractor import SequenceFeatureExtractor
from fairseq2_b200.models.transformer.frontend import TransformerFrontend
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.position_encoder import PositionEncoder
from fairseq2_b200.nn.projection import Projection
from fairseq2_b200.typing import DataType, Device


class Conv1dFbankSubsampler(SequenceFeatureExtractor):
    STRIDE = 2

    def __init__(self, num_channels: int, inner_dim: int, feature_dim: int, *,
                 kernel_sizes: Sequence[int] | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(feature_dim)
        kernel_sizes = list(kernel_sizes) if kernel_sizes is not None else [3, 3]
        self.layers = Sequential()
        last = len(kernel_sizes) - 1
        for i, k in enumerate(kernel_sizes):
            layer = Sequential()
            in_dim = num_channels if i == 0 else inner_dim // 2
            out_dim = feature_dim * 2 if i == last else inner_dim
            layer.add_module("conv", Conv1d(in_dim, out_dim, k, stride=self.STRIDE, padding=k // 2, device=device,
                                            dtype=dtype))
            layer.add_module("activation", GLU(dim=1))
            self.layers.append(layer)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout]:
        if seqs_layout.packed:
            raise ValueError("`seqs` must not be a packed batch.")
        seqs = self.layers(seqs.transpose(1, 2)).transpose(1, 2)
        lens = list(seqs_layout.seq_lens)
        for _ in range(len(self.layers)):
            lens = [int(math.floor((n - 1) / self.STRIDE + 1.0)) for n in lens]
        return seqs, BatchLayout(tuple(seqs.shape[:2]), lens, device=seqs.device)


class S2TTransformerFrontend(TransformerFrontend):
    def __init__(self, model_dim: int, feature_extractor: SequenceFeatureExtractor | None,
                 pos_encoder: PositionEncoder | None, proj: Projection | None, *, dropout_p: float = 0.0) -> None:
        super().__init__()
        self.model_dim = model_dim
        self.feature_extractor = feature_extractor
        self.scale = math.sqrt(model_dim)
        self.pos_encoder = pos_encoder
        self.proj = proj
        self.dropout = Dropout(dropout_p) if dropout_p > 0.0 else None

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None  # type: ignore[override]
                ) -> tuple[Tensor, BatchLayout]:
        if state_bag is not None:
            raise NotSupportedError("`S2TTransformerFrontend` does not support incremental decoding.")
        if self.feature_extractor is not None:
            seqs, seqs_layout = self.feature_extractor(seqs, seqs_layout)
        seqs = seqs * self.scale
        if self.pos_encoder is not None:
            seqs = self.pos_encoder(seqs, seqs_layout)
        if self.proj is not None:
            seqs = self.proj(seqs)
        if self.dropout is not None:
            seqs = self.dropout(seqs)
        return seqs, seqs_layout
