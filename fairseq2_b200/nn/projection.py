"""Linear projections, including the tensor-parallel variants.

Capability parity with fairseq2 ``nn/projection.py`` (``Linear`` :59,
``ColumnShardedLinear`` :128, ``RowShardedLinear`` :365, ``TiedProjection``
:600, ``IdentityProjection`` :618). All matrix products go through
``fairseq2_b200.ops.gemm.linear`` (tcgen05 GEMM on CUDA).

The sharded linears additionally offer a *sequence-parallel* mode
(``sequence_parallel=True``): the column linear all-gathers a sequence-sharded
input and the row linear reduce-scatters its output, which halves TP traffic
relative to the all-reduce pair and removes the redundant norm/residual work.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Callable

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.gang import Gang
from fairseq2_b200.ops.gemm import linear as _linear
from fairseq2_b200.ops.tensor_parallel import (all_gather_seq, gather, reduce, reduce_on_backward,
                                               reduce_scatter_seq, scatter)
from fairseq2_b200.typing import DataType, Device


def _fused_ops(gang: Gang, x: Tensor, rows: int, model_dim: int, weight: Tensor):  # type: ignore[no-untyped-def]
    """The fused all-gather / reduce-scatter GEMM operators for token shards of ``rows x model_dim``, if the call
    is one the sm_100a kernels cover (bf16 on CUDA, 2-D activations, tile-aligned shard) and the gang has a
    symmetric arena; ``None`` otherwise (the caller then uses the gang's collectives)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.ndim == 2 and weight.dtype == torch.bfloat16):
        return None
    from fairseq2_b200.ops._ext import use_kernels

    if not use_kernels(x):
        return None
    from fairseq2_b200.parallel.tp import get_tp_context

    return get_tp_context(gang).linears(x, rows, model_dim)


class Projection(Module, ABC):
    def __init__(self, input_dim: int, output_dim: int) -> None:
        super().__init__()
        self.input_dim, self.output_dim = input_dim, output_dim

    @abstractmethod
    def forward(self, x: Tensor) -> Tensor: ...


def _default_linear_init(weight: Tensor, bias: Tensor | None) -> None:
    torch.nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
    if bias is not None:
        fan_in = weight.shape[1]
        bound = 1.0 / math.sqrt(fan_in) if fan_in > 0 else 0.0
        torch.nn.init.uniform_(bias, -bound, bound)


class Linear(Projection):
    def __init__(self, input_dim: int, output_dim: int, bias: bool, *,
                 init_fn: Callable[["Linear"], None] | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(input_dim, output_dim)
        self.weight = Parameter(torch.empty((output_dim, input_dim), device=device, dtype=dtype))
        if bias:
            self.bias = Parameter(torch.empty((output_dim,), device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.init_fn = init_fn
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.init_fn is not None:
            self.init_fn(self)
        else:
            _default_linear_init(self.weight, self.bias)

    def forward(self, x: Tensor) -> Tensor:
        return _linear(x, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"input_dim={self.input_dim}, output_dim={self.output_dim}, bias={self.bias is not None}"


def _init_full_then_shard(kls: type, input_dim: int, output_dim: int, bias: bool, init_fn, gang: Gang, dim: int,
                          weight: Tensor, bias_t: Tensor | None) -> None:
    """Sharded layers are initialised as the matching slice of the full,
    unsharded initialisation so a TP model equals its single-rank counterpart."""
    if weight.device.type == "meta":
        return
    full = Linear(input_dim, output_dim, bias, init_fn=init_fn, device=weight.device, dtype=weight.dtype)
    with torch.no_grad():
        c = full.weight.shape[dim] // gang.size
        weight.copy_(full.weight.narrow(dim, gang.rank * c, c))
        if bias_t is not None and full.bias is not None:
            if dim == 0:
                bias_t.copy_(full.bias.narrow(0, gang.rank * c, c))
            else:
                bias_t.copy_(full.bias)


class ColumnShardedLinear(Projection):
    """``W`` split along the output dimension over ``gang``.

    fwd: (all-reduce the input gradient on bwd) -> local GEMM -> optional
    all-gather of the output features.
    """

    def __init__(self, gang: Gang, input_dim: int, output_dim: int, bias: bool, *, gather_output: bool = True,
                 sequence_parallel: bool = False, init_fn: Callable[[Linear], None] | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(input_dim, output_dim)
        if output_dim % gang.size:
            raise ValueError(f"`output_dim` must be a multiple of `gang.size` ({gang.size}), but is {output_dim} instead.")
        self.gang, self.gather_output, self.sequence_parallel = gang, gather_output, sequence_parallel
        self.sharded_output_dim = output_dim // gang.size
        self.weight = Parameter(torch.empty((self.sharded_output_dim, input_dim), device=device, dtype=dtype))
        if bias:
            self.bias = Parameter(torch.empty((self.sharded_output_dim,), device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.init_fn = init_fn
        self.reset_parameters()

    @staticmethod
    def from_linear(linear: Linear, gang: Gang, gather_output: bool = True) -> "ColumnShardedLinear":
        dev = linear.weight.device
        m = ColumnShardedLinear(gang, linear.input_dim, linear.output_dim, linear.bias is not None,
                                gather_output=gather_output, init_fn=linear.init_fn, device=torch.device("meta"),
                                dtype=linear.weight.dtype)
        m.to_empty(device=dev)
        with torch.no_grad():
            c = m.sharded_output_dim
            m.weight.copy_(linear.weight[gang.rank * c:(gang.rank + 1) * c])
            if m.bias is not None:
                m.bias.copy_(linear.bias[gang.rank * c:(gang.rank + 1) * c])
        return m

    def reset_parameters(self) -> None:
        _init_full_then_shard(Linear, self.input_dim, self.output_dim, self.bias is not None, self.init_fn, self.gang,
                              0, self.weight, self.bias)

    def forward(self, x: Tensor) -> Tensor:
        if self.sequence_parallel and self.gang.size > 1:
            # x is this rank's token shard [T / W, D]: the all-gather of the tokens runs inside the GEMM
            ops = _fused_ops(self.gang, x, x.shape[0] if x.ndim == 2 else 0, self.input_dim, self.weight)
            if ops is not None and self.bias is None and not self.gather_output:
                return ops.column(x, self.weight)
            x = all_gather_seq(x, self.gang, dim=-2)
        else:
            x = reduce_on_backward(x, self.gang)
        y = _linear(x, self.weight, self.bias)
        if self.gather_output:
            y = gather(y, self.gang, dim=-1)
        return y

    def to_linear(self, device: Device | None = None) -> Linear:
        full_w = gather(self.weight.detach(), self.gang, dim=0)
        lin = Linear(self.input_dim, self.output_dim, self.bias is not None, device=torch.device("meta"),
                     dtype=self.weight.dtype)
        lin.to_empty(device=device or self.weight.device)
        with torch.no_grad():
            lin.weight.copy_(full_w)
            if self.bias is not None:
                lin.bias.copy_(gather(self.bias.detach(), self.gang, dim=0))
        return lin

    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        out = [(self.weight, 0)]
        if self.bias is not None:
            out.append((self.bias, 0))
        return out

    def extra_repr(self) -> str:
        return (f"tp_rank={self.gang.rank}, tp_size={self.gang.size}, input_dim={self.input_dim}, "
                f"output_dim={self.output_dim}, sharded_output_dim={self.sharded_output_dim}, "
                f"gather_output={self.gather_output}, bias={self.bias is not None}")


class RowShardedLinear(Projection):
    """``W`` split along the input dimension over ``gang``.

    fwd: optional scatter of the input features -> local GEMM -> all-reduce
    (or reduce-scatter over the sequence in sequence-parallel mode) -> + bias.
    """

    def __init__(self, gang: Gang, input_dim: int, output_dim: int, bias: bool, *, scatter_input: bool = True,
                 sequence_parallel: bool = False, init_fn: Callable[[Linear], None] | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(input_dim, output_dim)
        if input_dim % gang.size:
            raise ValueError(f"`input_dim` must be a multiple of `gang.size` ({gang.size}), but is {input_dim} instead.")
        self.gang, self.scatter_input, self.sequence_parallel = gang, scatter_input, sequence_parallel
        self.sharded_input_dim = input_dim // gang.size
        self.weight = Parameter(torch.empty((output_dim, self.sharded_input_dim), device=device, dtype=dtype))
        if bias:
            self.bias = Parameter(torch.empty((output_dim,), device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.init_fn = init_fn
        self.reset_parameters()

    @staticmethod
    def from_linear(linear: Linear, gang: Gang, scatter_input: bool = False) -> "RowShardedLinear":
        dev = linear.weight.device
        m = RowShardedLinear(gang, linear.input_dim, linear.output_dim, linear.bias is not None,
                             scatter_input=scatter_input, init_fn=linear.init_fn, device=torch.device("meta"),
                             dtype=linear.weight.dtype)
        m.to_empty(device=dev)
        with torch.no_grad():
            c = m.sharded_input_dim
            m.weight.copy_(linear.weight[:, gang.rank * c:(gang.rank + 1) * c])
            if m.bias is not None:
                m.bias.copy_(linear.bias)
        return m

    def reset_parameters(self) -> None:
        _init_full_then_shard(Linear, self.input_dim, self.output_dim, self.bias is not None, self.init_fn, self.gang,
                              1, self.weight, self.bias)

    def forward(self, x: Tensor) -> Tensor:
        if self.scatter_input:
            x = scatter(x, self.gang, dim=-1)
        if self.sequence_parallel and self.gang.size > 1:
            # the GEMM epilogue sends every output tile to the rank that owns its tokens: y is [T / W, D]
            rows = x.shape[0] // self.gang.size if x.ndim == 2 and x.shape[0] % self.gang.size == 0 else 0
            ops = _fused_ops(self.gang, x, rows, self.output_dim, self.weight)
            if ops is not None:
                y = ops.row(x if x.is_contiguous() else x.contiguous(), self.weight)
            else:
                y = reduce_scatter_seq(_linear(x, self.weight, None), self.gang, dim=-2)
        else:
            y = reduce(_linear(x, self.weight, None), self.gang)
        if self.bias is not None:
            y = y + self.bias
        return y

    def to_linear(self, device: Device | None = None) -> Linear:
        full_w = gather(self.weight.detach(), self.gang, dim=1)
        lin = Linear(self.input_dim, self.output_dim, self.bias is not None, device=torch.device("meta"),
                     dtype=self.weight.dtype)
        lin.to_empty(device=device or self.weight.device)
        with torch.no_grad():
            lin.weight.copy_(full_w)
            if self.bias is not None:
                lin.bias.copy_(self.bias)
        return lin

    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        return [(self.weight, 1)]

    def extra_repr(self) -> str:
        return (f"tp_rank={self.gang.rank}, tp_size={self.gang.size}, input_dim={self.input_dim}, "
                f"sharded_input_dim={self.sharded_input_dim}, output_dim={self.output_dim}, "
                f"scatter_input={self.scatter_input}, bias={self.bias is not None}")


class TiedProjection(Projection):
    """Projects with a weight owned by another module (e.g. the embedding table)."""

    def __init__(self, weight: Parameter, bias: Parameter | None = None) -> None:
        super().__init__(weight.shape[1], weight.shape[0])
        self.weight, self.bias = weight, bias

    def forward(self, x: Tensor) -> Tensor:
        return _linear(x, self.weight, self.bias)


class IdentityProjection(Projection):
    def __init__(self, dim: int) -> None:
        super().__init__(dim, dim)

    def forward(self, x: Tensor) -> Tensor:
        return x


def init_bert_projection(proj: Linear) -> None:
    """Normal(0, 0.02) weights, zero bias (BERT / wav2vec2 encoder init)."""
    torch.nn.init.normal_(proj.weight, mean=0.0, std=0.02)
    if proj.bias is not None:
        torch.nn.init.zeros_(proj.bias)
