"""wav2vec 2.0 feature extractors (cf. fairseq2 ``models/wav2vec2/feature_extractor.py:34-377``).

The waveform extractor is a stack of strided 1-D convolutions, each followed by
dropout, a normalisation (group norm on the first layer, or layer norm on every
layer) and GELU. Activations stay channels-first through the whole stack; the
gradient flowing back into the extractor can be scaled down.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
from torch import Tensor
from torch.nn import GELU, Conv1d, Dropout, GroupNorm, Module, ModuleList

from fairseq2_b200.models.feature_extractor import SequenceFeatureExtractor
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.normalization import StandardLayerNorm
from fairseq2_b200.typing import DataType, Device


class _ScaleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, scale: float) -> Tensor:  # type: ignore[override]
        ctx.scale = scale
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return g * ctx.scale, None


def scale_gradient(x: Tensor, scale: float) -> Tensor:
    """Identity in forward; multiplies the gradient by ``scale`` in backward."""
    return _ScaleGrad.apply(x, scale)


class Float32GroupNorm(GroupNorm):
    def forward(self, x: Tensor) -> Tensor:
        w = self.weight.float() if self.weight is not None else None
        b = self.bias.float() if self.bias is not None else None
        return torch.nn.functional.group_norm(x.float(), self.num_groups, w, b, self.eps).type_as(x)


class Wav2Vec2FeatureConv1d(Conv1d):
    def reset_parameters(self) -> None:
        if self.weight.device.type == "meta":
            return
        torch.nn.init.kaiming_normal_(self.weight)
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)


class Wav2Vec2FeatureExtractionLayer(Module):
    def __init__(self, input_dim: int, output_dim: int, kernel_size: int, stride: int, bias: bool, *,
                 dropout_p: float = 0.0, group_norm: GroupNorm | None = None,
                 layer_norm: StandardLayerNorm | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__()
        self.conv = Wav2Vec2FeatureConv1d(input_dim, output_dim, kernel_size, stride=stride, bias=bias, device=device,
                                          dtype=dtype)
        self.dropout = Dropout(dropout_p) if dropout_p > 0.0 else None
        self.group_norm, self.layer_norm = group_norm, layer_norm
        self.activation = GELU()

    def forward(self, seqs: Tensor) -> Tensor:
        seqs = self.conv(seqs)                       # (N, C, S)
        if self.dropout is not None:
            seqs = self.dropout(seqs)
        if self.group_norm is not None:
            seqs = self.group_norm(seqs)
        if self.layer_norm is not None:
            seqs = self.layer_norm(seqs.transpose(1, 2)).transpose(1, 2)
        return self.activation(seqs)


class Wav2Vec2FeatureExtractor(SequenceFeatureExtractor):
    """``layer_descs``: ``(output_dim, kernel_size, stride)`` per convolution."""

    def __init__(self, layer_descs: Sequence[tuple[int, int, int]], bias: bool, *, num_channels: int = 1,
                 dropout_p: float = 0.0, layer_norm: bool = False, grad_scale: float = 1.0,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        if not layer_descs:
            raise ValueError("`layer_descs` must be non-empty.")
        super().__init__(layer_descs[-1][0])
        if not 0.0 < grad_scale <= 1.0:
            raise ValueError(f"`grad_scale` must be in (0, 1], but is {grad_scale} instead.")
        self.layer_descs = [tuple(d) for d in layer_descs]
        self.num_channels, self.grad_scale = num_channels, grad_scale
        layers = []
        in_dim = num_channels
        for i, (out_dim, k, s) in enumerate(self.layer_descs):
            gn = ln = None
            if layer_norm:
                ln = StandardLayerNorm(out_dim, bias=True, cast_fp32=True, device=device, dtype=dtype)
            elif i == 0:
                gn = Float32GroupNorm(out_dim, out_dim, device=device, dtype=dtype)
            layers.append(Wav2Vec2FeatureExtractionLayer(in_dim, out_dim, k, s, bias, dropout_p=dropout_p,
                                                         group_norm=gn, layer_norm=ln, device=device, dtype=dtype))
            in_dim = out_dim
        self.layers = ModuleList(layers)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout]:
        """``seqs``: ``(N, S)`` waveform or ``(N, S, C)`` multi-channel audio."""
        if seqs_layout.packed:
            raise ValueError("`seqs` must not be a packed batch.")
        x = seqs.unsqueeze(1) if self.num_channels == 1 and seqs.ndim == 2 else seqs.transpose(1, 2)
        if self._channels_last_ok(x):
            x = self._forward_channels_last(x)
            if self.training and self.grad_scale != 1.0:
                x = scale_gradient(x, self.grad_scale)
        else:
            for layer in self.layers:
                x = layer(x)
            if self.training and self.grad_scale != 1.0:
                x = scale_gradient(x, self.grad_scale)
            x = x.transpose(1, 2)                    # (N, S_out, C)
        lens = self._contract_seq_lens(seqs_layout.seq_lens)
        return x, BatchLayout(tuple(x.shape[:2]), lens, device=x.device)

    def _channels_last_ok(self, x: Tensor) -> bool:
        from fairseq2_b200.ops._ext import use_kernels

        if not (use_kernels(x) and x.dtype == torch.bfloat16 and len(self.layers) > 1):
            return False
        first = self.layers[0]
        if first.conv.weight.dtype != torch.bfloat16 or first.conv.out_channels % 8:
            return False
        return all(layer.conv.out_channels % 8 == 0 and layer.conv.kernel_size[0] >= layer.conv.stride[0]
                   and layer.group_norm is None for layer in self.layers[1:])

    def _forward_channels_last(self, x: Tensor) -> Tensor:
        """The first layer (one input channel) is one fused kernel when it has a LayerNorm, else it runs as usual;
        from then on activations stay channels-last
        ``(N, S, C)`` and every strided convolution is one tcgen05 GEMM over an overlapping-row view, followed by
        one fused LayerNorm+GELU kernel. Time steps are padded once so that every stride divides evenly; rows
        past the true output length are meaningless and cut off at the end."""
        from fairseq2_b200.ops.conv import conv1d_channels_last
        from fairseq2_b200.ops.norm import layer_norm_gelu

        from fairseq2_b200.ops.conv import first_conv_ln_gelu, first_conv_supported

        first = self.layers[0]
        valid = (x.shape[-1] - first.conv.kernel_size[0]) // first.conv.stride[0] + 1
        total_stride = 1
        for layer in self.layers[1:]:
            total_stride *= layer.conv.stride[0]
        pad = (-valid) % total_stride
        wave = x[:, 0] if x.shape[1] == 1 else None
        if (wave is not None and first.group_norm is None and first.layer_norm is not None
                and first.layer_norm.weight is not None and first.layer_norm.bias is not None
                and (first.dropout is None or not self.training or first.dropout.p == 0.0)
                and first_conv_supported(wave, first.conv.weight)):
            # one kernel: waveform -> conv + bias -> LayerNorm over the channels -> GELU -> channels-last, padded
            ln = first.layer_norm
            x = first_conv_ln_gelu(wave, first.conv.weight, first.conv.bias, ln.weight, ln.bias,
                                   first.conv.stride[0], valid + pad, ln.eps)
        else:
            x = first(x)                             # (N, C, S1)
            x = x.transpose(1, 2)
            x = torch.nn.functional.pad(x, (0, 0, 0, pad)) if pad else x.contiguous()
        for layer in self.layers[1:]:
            k, s = layer.conv.kernel_size[0], layer.conv.stride[0]
            x = conv1d_channels_last(x, layer.conv.weight, layer.conv.bias, s)
            valid = (valid - k) // s + 1
            if layer.dropout is not None:
                x = layer.dropout(x)
            if layer.layer_norm is not None:
                ln = layer.layer_norm
                x = layer_norm_gelu(x, ln.weight, ln.bias, ln.eps)
            else:
                x = torch.nn.functional.gelu(x)
        return x[:, :valid]

    def _contract_seq_lens(self, seq_lens: Sequence[int]) -> list[int]:
        out = list(seq_lens)
        for _, k, s in self.layer_descs:
            out = [int(math.floor((n - k) / s + 1.0)) for n in out]
        return out

    def extra_repr(self) -> str:
        return f"feature_dim={self.feature_dim}, grad_scale={self.grad_scale:G}"


class Wav2Vec2FbankFeatureExtractor(SequenceFeatureExtractor):
    """Stacks ``stride`` consecutive filter-bank frames into one feature vector."""

    def __init__(self, num_fbank_channels: int, stride: int, *, sample_every_k: int = 1) -> None:
        super().__init__(num_fbank_channels * stride)
        self.num_fbank_channels, self.stride, self.sample_every_k = num_fbank_channels, stride, sample_every_k

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout]:
        n, frames, ch = seqs.shape
        if ch != self.num_fbank_channels:
            raise ValueError(f"The last dimension of `seqs` must be {self.num_fbank_channels}, but is {ch} instead.")
        r = frames % self.stride
        if r:
            frames -= r
            seqs = seqs[:, :frames]
        seqs = seqs.reshape(n, frames // self.stride, ch * self.stride)
        lens = [min(l, frames) // self.stride for l in seqs_layout.seq_lens]
        if self.sample_every_k > 1:
            idx = torch.arange(0, seqs.shape[1], device=seqs.device)
            seqs = seqs[:, idx[idx % self.sample_every_k != 0]]
            lens = [l - (l + self.sample_every_k - 1) // self.sample_every_k for l in lens]
        return seqs, BatchLayout(tuple(seqs.shape[:2]), lens, device=seqs.device)
