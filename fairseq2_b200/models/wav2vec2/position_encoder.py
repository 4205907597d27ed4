"""Convolutional position encoders of wav2vec 2.0 (cf. fairseq2 ``models/wav2vec2/position_encoder.py:32-289``)."""
from __future__ import annotations

import torch
from torch import Tensor
from torch.nn import GELU, Conv1d, Module, Sequential
from torch.nn.utils.parametrizations import weight_norm

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.normalization import StandardLayerNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder
from fairseq2_b200.nn.utils.mask import apply_mask
from fairseq2_b200.typing import DataType, Device


class Wav2Vec2PositionalConv1d(Conv1d):
    def reset_parameters(self) -> None:
        from torch.nn.utils import parametrize

        model_dim, kernel_size = self.in_channels, self.kernel_size[0]
        std = (4.0 / (kernel_size * model_dim)) ** 0.5
        if parametrize.is_parametrized(self, "weight"):
            # weight-normalised: ``self.weight`` is computed from (magnitude, direction); a fresh weight has to be
            # assigned so that the parametrisation's right inverse refills both (an in-place init of the computed
            # tensor would be lost -- this is the path taken when the module was built on the meta device)
            direction = self.parametrizations.weight.original1
            if direction.device.type == "meta":
                return
            with torch.no_grad():
                self.weight = torch.empty_like(direction).normal_(mean=0.0, std=std)
        else:
            if self.weight.device.type == "meta":
                return
            torch.nn.init.normal_(self.weight, mean=0.0, std=std)
        if self.bias is not None and self.bias.device.type != "meta":
            torch.nn.init.zeros_(self.bias)


def _zero_padding(seqs: Tensor, layout: BatchLayout) -> Tensor:
    if not layout.padded:
        return seqs
    return apply_mask(seqs, layout.position_indices >= 0)


class Wav2Vec2PositionEncoder(PositionEncoder):
    """``x + GELU(grouped_conv(x))`` with a weight-normalised, same-padded convolution."""

    def __init__(self, model_dim: int, kernel_size: int, num_groups: int, *, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(model_dim)
        conv = Wav2Vec2PositionalConv1d(model_dim, model_dim, kernel_size, padding=kernel_size // 2, groups=num_groups,
                                        device=device, dtype=dtype)
        self.conv = weight_norm(conv, dim=2)
        self.remove_pad = kernel_size % 2 == 0
        self.activation = GELU()

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        if state_bag is not None:
            raise ValueError("`Wav2Vec2PositionEncoder` does not support incremental decoding.")
        seqs = _zero_padding(seqs, seqs_layout)      # padding must not leak into the convolution
        from fairseq2_b200.ops.conv import grouped_conv1d_channels_last, grouped_conv1d_supported

        conv = self.conv
        weight = conv.weight                         # evaluates the weight-norm parametrisation once
        if grouped_conv1d_supported(seqs, weight, conv.groups):
            # channels-last all the way: one tcgen05 GEMM per group over an overlapping-row view
            enc = grouped_conv1d_channels_last(seqs, weight, conv.bias, conv.groups, conv.padding[0])
            if self.remove_pad:
                enc = enc[:, :-1]
            return seqs + self.activation(enc)
        enc = torch.nn.functional.conv1d(seqs.transpose(1, 2), weight, conv.bias, padding=conv.padding[0],
                                         groups=conv.groups)
        if self.remove_pad:
            enc = enc[:, :, :-1]
        return seqs + self.activation(enc).transpose(1, 2)


class Wav2Vec2StackedPositionEncoder(PositionEncoder):
    """``depth`` smaller grouped convolutions, each followed by a parameter-free layer norm and GELU."""

    def __init__(self, model_dim: int, kernel_size: int, num_groups: int, num_layers: int, *,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(model_dim)
        k = max(3, kernel_size // num_layers)
        self.layers = Sequential(*[_StackedLayer(model_dim, k, num_groups, device, dtype) for _ in range(num_layers)])

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        if state_bag is not None:
            raise ValueError("`Wav2Vec2StackedPositionEncoder` does not support incremental decoding.")
        seqs = _zero_padding(seqs, seqs_layout)
        return seqs + self.layers(seqs.transpose(1, 2)).transpose(1, 2)


class _StackedLayer(Module):
    def __init__(self, model_dim: int, kernel_size: int, num_groups: int, device: Device | None,
                 dtype: DataType | None) -> None:
        super().__init__()
        self.conv = Conv1d(model_dim, model_dim, kernel_size, padding="same", groups=num_groups, device=device,
                           dtype=dtype)
        self.layer_norm = StandardLayerNorm(model_dim, bias=False, elementwise_affine=False)
        self.activation = GELU()

    def forward(self, x: Tensor) -> Tensor:
        x = self.conv(x)
        x = self.layer_norm(x.transpose(1, 2)).transpose(1, 2)
        return self.activation(x)
