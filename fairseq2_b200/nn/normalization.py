"""Layer normalisation modules (cf. fairseq2 ``nn/normalization.py:49-269``).

Forward math is delegated to ``fairseq2_b200.ops.norm`` which runs the
hand-written sm_100a kernels on CUDA tensors.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable, Sequence

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.ops import norm as _norm_ops
from fairseq2_b200.typing import DataType, Device


class LayerNorm(Module, ABC):
    normalized_shape: tuple[int, ...]
    eps: float
    elementwise_affine: bool

    def __init__(self, normalized_shape: int | Sequence[int], bias: bool, *, eps: float = 1e-5,
                 elementwise_affine: bool = True, init_fn: Callable[["LayerNorm"], None] | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = Parameter(torch.empty(self.normalized_shape, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        if elementwise_affine and bias:
            self.bias = Parameter(torch.empty(self.normalized_shape, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.init_fn = init_fn
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.init_fn is not None:
            self.init_fn(self)
            return
        if self.weight is not None:
            torch.nn.init.ones_(self.weight)
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)

    @abstractmethod
    def forward(self, x: Tensor) -> Tensor: ...

    @abstractmethod
    def apply_with(self, x: Tensor, weight: Tensor | None, bias: Tensor | None) -> Tensor:
        """The same normalisation with ``weight`` / ``bias`` given by the caller instead of the module's own
        (tensor-parallel callers pass the parameters through an identity whose backward sums over the gang)."""

    def extra_repr(self) -> str:
        s = f"normalized_shape={self.normalized_shape}, eps={self.eps:G}, elementwise_affine={self.elementwise_affine}"
        return s


class StandardLayerNorm(LayerNorm):
    def __init__(self, *a, cast_fp32: bool = False, **kw) -> None:  # type: ignore[no-untyped-def]
        self.cast_fp32 = cast_fp32
        super().__init__(*a, **kw)

    def forward(self, x: Tensor) -> Tensor:
        return self.apply_with(x, self.weight, self.bias)

    def apply_with(self, x: Tensor, weight: Tensor | None, bias: Tensor | None) -> Tensor:
        return _norm_ops.layer_norm(x, self.normalized_shape, weight, bias, self.eps, cast_fp32=self.cast_fp32)


class RMSNorm(LayerNorm):
    """Root-mean-square norm: ``x * rsqrt(mean(x^2) + eps) * w``, statistics in fp32."""

    def forward(self, x: Tensor) -> Tensor:
        return self.apply_with(x, self.weight, self.bias)

    def apply_with(self, x: Tensor, weight: Tensor | None, bias: Tensor | None) -> Tensor:
        return _norm_ops.rms_norm(x, self.normalized_shape, weight, self.eps, bias=bias)
