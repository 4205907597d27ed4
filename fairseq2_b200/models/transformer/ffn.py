"""Feed-forward networks (cf. fairseq2 ``models/transformer/ffn.py``:
standard :43, Dauphin :135, GLU :229, AltUp :407).

``GLUFeedForwardNetwork`` runs gate and up projections as ONE GEMM whenever
their weights are adjacent in memory and applies ``silu(gate) * up`` with the
fused SwiGLU kernel.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Callable

import torch
from torch import Tensor
from torch.nn import Dropout, Module, ReLU, SiLU

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.gang import Gang, Gangs
from fairseq2_b200.models.transformer.multihead_attention import merged_linear
from fairseq2_b200.nn.normalization import LayerNorm
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, Projection, RowShardedLinear
from fairseq2_b200.ops.activation import swiglu
from fairseq2_b200.typing import DataType, Device


class FeedForwardNetwork(Module, ABC):
    def __init__(self, model_dim: int) -> None:
        super().__init__()
        self.model_dim = model_dim

    @abstractmethod
    def forward(self, seqs: Tensor) -> Tensor: ...


def _col(gangs: Gangs | None, i: int, o: int, bias: bool, init_fn, device, dtype) -> Projection:  # type: ignore[no-untyped-def]
    if gangs is not None and gangs.tp.size > 1:
        from fairseq2_b200.parallel.tp import sequence_parallel_enabled

        return ColumnShardedLinear(gangs.tp, i, o, bias, gather_output=False,
                                   sequence_parallel=sequence_parallel_enabled(), init_fn=init_fn, device=device,
                                   dtype=dtype)
    return Linear(i, o, bias, init_fn=init_fn, device=device, dtype=dtype)


def _row(gangs: Gangs | None, i: int, o: int, bias: bool, init_fn, device, dtype) -> Projection:  # type: ignore[no-untyped-def]
    if gangs is not None and gangs.tp.size > 1:
        from fairseq2_b200.parallel.tp import sequence_parallel_enabled

        return RowShardedLinear(gangs.tp, i, o, bias, scatter_input=False,
                                sequence_parallel=sequence_parallel_enabled(), init_fn=init_fn, device=device,
                                dtype=dtype)
    return Linear(i, o, bias, init_fn=init_fn, device=device, dtype=dtype)


class StandardFeedForwardNetwork(FeedForwardNetwork):
    def __init__(self, model_dim: int, inner_dim: int, bias: bool, *, inner_activation: Module | None = None,
                 inner_dropout_p: float = 0.0, inner_layer_norm: LayerNorm | None = None,
                 proj_init_fn: Callable[[Linear], None] | None = None, gangs: Gangs | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(model_dim)
        if inner_layer_norm is not None and gangs is not None and gangs.tp.size > 1:
            # the norm spans the inner dimension, which tensor parallelism splits over the ranks
            raise NotSupportedError("`inner_layer_norm` is not supported when tensor parallelism is enabled.")
        self.inner_proj = _col(gangs, model_dim, inner_dim, bias, proj_init_fn, device, dtype)
        self.inner_activation = inner_activation if inner_activation is not None else ReLU()
        self.inner_dropout = Dropout(inner_dropout_p) if inner_dropout_p > 0.0 else None
        self.inner_layer_norm = inner_layer_norm
        self.output_proj = _row(gangs, inner_dim, model_dim, bias, proj_init_fn, device, dtype)

    def forward(self, seqs: Tensor) -> Tensor:
        seqs = self.inner_activation(self.inner_proj(seqs))
        if self.inner_layer_norm is not None:
            seqs = self.inner_layer_norm(seqs)
        if self.inner_dropout is not None:
            seqs = self.inner_dropout(seqs)
        return self.output_proj(seqs)


class DauphinFeedForwardNetwork(FeedForwardNetwork):
    """GLU of Dauphin et al.: one projection to ``2·inner``, ``a * sigmoid(b)``."""

    def __init__(self, model_dim: int, inner_dim: int, bias: bool, *, inner_activation: Module | None = None,
                 inner_dropout_p: float = 0.0, device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(model_dim)
        self.inner_proj = Linear(model_dim, inner_dim * 2, bias, device=device, dtype=dtype)
        self.inner_activation = inner_activation if inner_activation is not None else torch.nn.Sigmoid()
        self.inner_dropout = Dropout(inner_dropout_p) if inner_dropout_p > 0.0 else None
        self.output_proj = Linear(inner_dim, model_dim, bias, device=device, dtype=dtype)

    def forward(self, seqs: Tensor) -> Tensor:
        a, b = self.inner_proj(seqs).chunk(2, dim=-1)
        seqs = a * self.inner_activation(b)
        if self.inner_dropout is not None:
            seqs = self.inner_dropout(seqs)
        return self.output_proj(seqs)


class GLUFeedForwardNetwork(FeedForwardNetwork):
    """``output_proj(act(gate_proj(x)) * inner_proj(x))`` (SwiGLU by default).

    ``inner_dim`` is scaled by ``inner_dim_scale`` (2/3 in LLaMA) and rounded up
    to a multiple of ``inner_dim_to_multiple``.
    """

    def __init__(self, model_dim: int, inner_dim: int, bias: bool, *, gate_activation: Module | None = None,
                 inner_dim_scale: float = 2 / 3, inner_dim_to_multiple: int = 1, inner_dropout_p: float = 0.0,
                 proj_init_fn: Callable[[Linear], None] | None = None, gangs: Gangs | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(model_dim)
        self.inner_dim_scale, self.inner_dim_to_multiple = inner_dim_scale, inner_dim_to_multiple
        if inner_dim_scale != 1.0:
            inner_dim = int(inner_dim * inner_dim_scale)
        if inner_dim_to_multiple != 1:
            inner_dim = inner_dim_to_multiple * ((inner_dim + inner_dim_to_multiple - 1) // inner_dim_to_multiple)
        self.inner_dim = inner_dim
        self.gate_proj = _col(gangs, model_dim, inner_dim, bias, proj_init_fn, device, dtype)
        self.gate_activation = gate_activation if gate_activation is not None else SiLU()
        self.inner_proj = _col(gangs, model_dim, inner_dim, bias, proj_init_fn, device, dtype)
        self.inner_dropout = Dropout(inner_dropout_p) if inner_dropout_p > 0.0 else None
        self.output_proj = _row(gangs, inner_dim, model_dim, bias, proj_init_fn, device, dtype)

    def forward(self, seqs: Tensor) -> Tensor:
        h = None
        if isinstance(self.gate_activation, SiLU):
            gu = merged_linear(seqs, [self.gate_proj, self.inner_proj])
            if gu is not None:
                h = swiglu(gu)
        if h is None:
            h = self.gate_activation(self.gate_proj(seqs)) * self.inner_proj(seqs)
        if self.inner_dropout is not None:
            h = self.inner_dropout(h)
        return self.output_proj(h)

    def extra_repr(self) -> str:
        return f"model_dim={self.model_dim}, inner_dim={self.inner_dim}"


def gaussian_topk(x: Tensor, sparsity: float, tp_gang: Gang | None = None, full_dim: int | None = None) -> Tensor:
    """Keeps roughly the top ``1 - sparsity`` fraction of every row: entries below ``mean + z * std`` (``z`` the
    standard-normal quantile of ``sparsity``) become zero, the rest are shifted down by that cut-off. With the last
    dimension split over ``tp_gang`` (``full_dim`` entries in total) the two moments are summed over the gang."""
    z = math.sqrt(2.0) * float(torch.erfinv(torch.tensor(2.0 * sparsity - 1.0)))
    if tp_gang is None or tp_gang.size == 1:
        mean = x.mean(dim=-1, keepdim=True)
        std = x.std(dim=-1, keepdim=True, unbiased=False)
    else:
        from fairseq2_b200.ops.tensor_parallel import reduce_both_ways

        n = full_dim if full_dim is not None else x.shape[-1] * tp_gang.size
        xf = x.float()
        moments = reduce_both_ways(torch.stack([xf.sum(-1), xf.pow(2).sum(-1)], dim=-1), tp_gang)
        mean = moments[..., :1] / n
        std = (moments[..., 1:] / n - mean.pow(2)).clamp_min(0.0).sqrt()
        mean, std = mean.type_as(x), std.type_as(x)
    return torch.nn.functional.relu(x - (mean + std * z))


class AltUpFeedForwardNetwork(FeedForwardNetwork):
    """Gated FFN of the Gemma 3n layers: ``output_proj(gelu_tanh(sparsify(gate_proj(x))) * inner_proj(x))`` where
    ``sparsify`` is :func:`gaussian_topk` when ``activation_sparsity`` > 0 (cf. fairseq2
    ``models/transformer/ffn.py:407-501``). Tensor parallel over the inner dimension when ``gangs.tp`` has more than
    one rank."""

    def __init__(self, model_dim: int, inner_dim: int, bias: bool, *, activation_sparsity: float = 0.0,
                 gangs: Gangs | None = None, device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(model_dim)
        if not 0.0 <= activation_sparsity < 1.0:
            raise ValueError(f"`activation_sparsity` must be in [0, 1), but is {activation_sparsity} instead.")
        self.inner_dim, self.activation_sparsity = inner_dim, activation_sparsity
        self.tp_gang = gangs.tp if gangs is not None and gangs.tp.size > 1 else None
        self.gate_proj = _col(gangs, model_dim, inner_dim, bias, None, device, dtype)
        self.inner_proj = _col(gangs, model_dim, inner_dim, bias, None, device, dtype)
        self.output_proj = _row(gangs, inner_dim, model_dim, bias, None, device, dtype)

    def forward(self, seqs: Tensor) -> Tensor:
        gate = self.gate_proj(seqs)
        if self.activation_sparsity > 0.0:
            gate = gaussian_topk(gate, self.activation_sparsity, self.tp_gang, self.inner_dim)
        return self.output_proj(torch.nn.functional.gelu(gate, approximate="tanh") * self.inner_proj(seqs))
