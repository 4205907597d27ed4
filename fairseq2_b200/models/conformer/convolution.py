"""Conformer convolution module (cf. fairseq2 ``models/conformer/convolution.py:26-183``):
pointwise conv -> GLU -> depthwise conv (optionally causal) -> batch/layer norm -> SiLU -> pointwise conv."""
from __future__ import annotations

from typing import Literal

from torch import Tensor
from torch.nn import GLU, BatchNorm1d, Conv1d, Module, SiLU
from torch.nn.functional import pad

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.normalization import StandardLayerNorm
from fairseq2_b200.nn.utils.mask import apply_mask
from fairseq2_b200.typing import DataType, Device


class ConformerConvolution(Module):
    def __init__(self, model_dim: int, depthwise_kernel_size: int, *, causal_depthwise_conv: bool = False,
                 norm_type: Literal["batch_norm", "layer_norm"] = "batch_norm",
                 depthwise_activation: Module | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__()
        if norm_type not in ("batch_norm", "layer_norm"):
            raise ValueError(f"`norm_type` must be 'batch_norm' or 'layer_norm', but is '{norm_type}' instead.")
        self.model_dim = model_dim
        kw = {"device": device, "dtype": dtype}
        self.pointwise_conv1 = Conv1d(model_dim, 2 * model_dim, 1, bias=False, **kw)
        self.pointwise_conv1_activation = GLU(dim=1)
        self.depthwise_conv = Conv1d(model_dim, model_dim, depthwise_kernel_size,
                                     padding=0 if causal_depthwise_conv else "same", groups=model_dim, bias=False,
                                     **kw)
        self.causal_depthwise_conv = causal_depthwise_conv
        self.batch_norm = BatchNorm1d(model_dim, **kw) if norm_type == "batch_norm" else None
        self.layer_norm = StandardLayerNorm(model_dim, bias=True, **kw) if norm_type == "layer_norm" else None
        self.depthwise_activation = depthwise_activation if depthwise_activation is not None else SiLU()
        self.pointwise_conv2 = Conv1d(model_dim, model_dim, 1, bias=False, **kw)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> Tensor:
        if seqs_layout.packed:
            raise ValueError("`seqs` must not be a packed batch.")
        if seqs_layout.padded:
            seqs = apply_mask(seqs, seqs_layout.position_indices >= 0)   # padding must not leak through the kernel
        x = seqs.transpose(1, 2)
        x = self.pointwise_conv1_activation(self.pointwise_conv1(x))
        if self.causal_depthwise_conv:
            x = pad(x, (self.depthwise_conv.kernel_size[0] - 1, 0))
        x = self.depthwise_conv(x)
        if self.batch_norm is not None:
            x = self.batch_norm(x)
        else:
            x = self.layer_norm(x.transpose(1, 2)).transpose(1, 2)
        x = self.pointwise_conv2(self.depthwise_activation(x))
        return x.transpose(1, 2)

    def extra_repr(self) -> str:
        return f"causal_depthwise_conv={self.causal_depthwise_conv}"
