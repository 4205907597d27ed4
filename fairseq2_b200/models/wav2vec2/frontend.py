"""wav2vec 2.0 encoder front end (cf. fairseq2 ``models/wav2vec2/frontend.py:32-223``): feature extraction,
feature layer norm, projection to the model dimension, masking, positional convolution, layer norm, dropout."""
from __future__ import annotations

from torch import Tensor
from torch.nn import Dropout

from fairseq2_b200.models.feature_extractor import SequenceFeatureExtractor
from fairseq2_b200.models.transformer.frontend import TransformerFrontend
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm, StandardLayerNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.typing import DataType, Device


class Wav2Vec2Frontend(TransformerFrontend):
    def __init__(self, model_dim: int, feature_dim: int, feature_extractor: SequenceFeatureExtractor | None,
                 pos_encoder: PositionEncoder | None, *, first_pass_dropout_p: float = 0.0, layer_norm: bool = False,
                 dropout_p: float = 0.0, device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__()
        self.model_dim, self.feature_dim = model_dim, feature_dim
        if feature_extractor is not None and feature_extractor.feature_dim != feature_dim:
            raise ValueError(f"`feature_dim` of `feature_extractor` must be {feature_dim}.")
        self.feature_extractor = feature_extractor
        self.post_extract_layer_norm = StandardLayerNorm(feature_dim, bias=True, device=device, dtype=dtype)
        self.model_dim_proj = Linear(feature_dim, model_dim, bias=True, device=device, dtype=dtype) \
            if feature_dim != model_dim else None
        self.first_pass_dropout = Dropout(first_pass_dropout_p) if first_pass_dropout_p > 0.0 else None
        self.pos_encoder = pos_encoder
        self.layer_norm: LayerNorm | None = StandardLayerNorm(model_dim, bias=True, device=device, dtype=dtype) \
            if layer_norm else None
        self.dropout = Dropout(dropout_p) if dropout_p > 0.0 else None

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None  # type: ignore[override]
                ) -> tuple[Tensor, BatchLayout]:
        if state_bag is not None:
            raise ValueError("`Wav2Vec2Frontend` does not support incremental decoding.")
        seqs, seqs_layout, _ = self.extract_features(seqs, seqs_layout)
        seqs, _ = self.process_features(seqs, seqs_layout)
        return seqs, seqs_layout

    def extract_features(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout, Tensor]:
        """Returns ``(normalised features, layout, raw features)``; the raw ones feed the feature penalty."""
        if self.feature_extractor is not None:
            seqs, seqs_layout = self.feature_extractor(seqs, seqs_layout)
        raw = seqs.clone()
        return self.post_extract_layer_norm(seqs), seqs_layout, raw

    def process_features(self, seqs: Tensor, seqs_layout: BatchLayout, masker: Wav2Vec2Masker | None = None
                         ) -> tuple[Tensor, Tensor | None]:
        if self.model_dim_proj is not None:
            seqs = self.model_dim_proj(seqs)
        if self.first_pass_dropout is not None:
            seqs = self.first_pass_dropout(seqs)
        mask = None
        if masker is not None:
            seqs, mask = masker(seqs, seqs_layout)
        if self.pos_encoder is not None:
            seqs = self.pos_encoder(seqs, seqs_layout)
        if self.layer_norm is not None:
            seqs = self.layer_norm(seqs)
        if self.dropout is not None:
            seqs = self.dropout(seqs)
        return seqs, mask
