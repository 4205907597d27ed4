"""Vision Transformer building blocks (cf. fairseq2 ``models/vit/feature_extractor.py:24-137``,
``models/vit/frontend.py:25-83``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable

from torch import Tensor
from torch.nn import Conv2d, Conv3d, Dropout, Module

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.models.transformer.frontend import TransformerFrontend
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.position_encoder import InterpolatedPositionEncoder
from fairseq2_b200.typing import DataType, Device


class PatchFeatureExtractor(Module, ABC):
    """``(N, C, *)`` images or videos -> ``(N, *grid, E)`` patch features."""

    @abstractmethod
    def forward(self, x: Tensor) -> Tensor: ...


class Conv2dPatchFeatureExtractor(PatchFeatureExtractor):
    def __init__(self, num_channels: int, feature_dim: int, patch_dims: tuple[int, int], *,
                 init_fn: Callable[[Conv2d], None] | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__()
        self.conv = Conv2d(num_channels, feature_dim, kernel_size=patch_dims, stride=patch_dims, device=device,
                           dtype=dtype)
        self.init_fn = init_fn
        if init_fn is not None and self.conv.weight.device.type != "meta":
            init_fn(self.conv)

    def forward(self, x: Tensor) -> Tensor:
        return self.conv(x).permute(0, 2, 3, 1)


class Conv3dPatchFeatureExtractor(PatchFeatureExtractor):
    def __init__(self, num_channels: int, feature_dim: int, patch_dims: tuple[int, int, int], *,
                 init_fn: Callable[[Conv3d], None] | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__()
        self.conv = Conv3d(num_channels, feature_dim, kernel_size=patch_dims, stride=patch_dims, device=device,
                           dtype=dtype)
        self.init_fn = init_fn
        if init_fn is not None and self.conv.weight.device.type != "meta":
            init_fn(self.conv)

    def forward(self, x: Tensor) -> Tensor:
        return self.conv(x).permute(0, 2, 3, 4, 1)


class StandardViTFrontend(TransformerFrontend):
    """Patchify, add interpolated grid positions, flatten the grid into a sequence."""

    def __init__(self, patch_feature_extractor: PatchFeatureExtractor, pos_encoder: InterpolatedPositionEncoder, *,
                 dropout_p: float = 0.0) -> None:
        super().__init__()
        self.patch_feature_extractor, self.pos_encoder = patch_feature_extractor, pos_encoder
        self.dropout = Dropout(dropout_p) if dropout_p > 0.0 else None

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None  # type: ignore[override]
                ) -> tuple[Tensor, BatchLayout]:
        if state_bag is not None:
            raise NotSupportedError("`StandardViTFrontend` does not support incremental decoding.")
        if seqs_layout.packed or seqs_layout.padded:
            raise ValueError("`seqs` must be neither a packed nor a padded batch.")
        x = self.pos_encoder(self.patch_feature_extractor(seqs))
        x = x.flatten(1, -2)
        if self.dropout is not None:
            x = self.dropout(x)
        return x, BatchLayout(tuple(x.shape[:2]), [x.shape[1]] * x.shape[0], device=x.device)
