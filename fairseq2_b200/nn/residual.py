"""Residual connection variants (cf. fairseq2 ``nn/residual.py:21-167``)."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch
from torch import Tensor
from torch.nn import Module


class ResidualConnect(Module, ABC):
    @abstractmethod
    def forward(self, seqs: Tensor, residual: Tensor) -> Tensor: ...


class AdditiveResidualConnect(ResidualConnect):
    def forward(self, seqs: Tensor, residual: Tensor) -> Tensor:
        return seqs + residual


class ScaledResidualConnect(ResidualConnect):
    def __init__(self, scale: float) -> None:
        super().__init__()
        self.scale = scale

    def forward(self, seqs: Tensor, residual: Tensor) -> Tensor:
        return seqs + self.scale * residual

    def extra_repr(self) -> str:
        return f"scale={self.scale}"


class DropPathResidualConnect(ResidualConnect):
    """Stochastic depth: the branch output of a whole sample is dropped with
    probability ``drop_p`` and survivors are scaled by ``1/(1-p)``."""

    def __init__(self, drop_p: float) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, seqs: Tensor, residual: Tensor) -> Tensor:
        if not self.training or self.drop_p == 0.0:
            return seqs + residual
        keep = 1.0 - self.drop_p
        shape = (seqs.shape[0],) + (1,) * (seqs.ndim - 1)
        mask = torch.empty(shape, dtype=seqs.dtype, device=seqs.device).bernoulli_(keep)
        return seqs * (mask / keep) + residual

    def extra_repr(self) -> str:
        return f"drop_p={self.drop_p}"


class LAuReLResidualConnect(ResidualConnect):
    """Learned augmented residual: ``seqs + residual + up(down(residual))``
    normalised (low-rank variant used by Gemma3n)."""

    def __init__(self, model_dim: int, rank: int, layer_norm: Module) -> None:
        super().__init__()
        from fairseq2_b200.nn.projection import Linear

        self.down = Linear(model_dim, rank, bias=False)
        self.up = Linear(rank, model_dim, bias=False)
        self.layer_norm = layer_norm

    def forward(self, seqs: Tensor, residual: Tensor) -> Tensor:
        low = self.layer_norm(self.up(self.down(residual)))
        return seqs + residual + low
