"""Embedding tables, including vocabulary- and dimension-sharded variants
(cf. fairseq2 ``nn/embedding.py``: ``StandardEmbedding`` :61,
``VocabShardedEmbedding`` :112, ``ShardedEmbedding`` :326)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.gang import Gang
from fairseq2_b200.ops.tensor_parallel import gather, reduce
from fairseq2_b200.typing import DataType, Device


class Embedding(Module, ABC):
    def __init__(self, num_embeddings: int, embed_dim: int, pad_idx: int | None) -> None:
        super().__init__()
        self.num_embeddings, self.embed_dim, self.pad_idx = num_embeddings, embed_dim, pad_idx

    @abstractmethod
    def forward(self, x: Tensor) -> Tensor: ...


def _default_embed_init(weight: Tensor, pad_idx: int | None) -> None:
    torch.nn.init.normal_(weight)
    if pad_idx is not None:
        with torch.no_grad():
            weight[pad_idx].fill_(0.0)


class StandardEmbedding(Embedding):
    def __init__(self, num_embeddings: int, embed_dim: int, pad_idx: int | None = None, *,
                 init_fn: Callable[["StandardEmbedding"], None] | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(num_embeddings, embed_dim, pad_idx)
        self.weight = Parameter(torch.empty((num_embeddings, embed_dim), device=device, dtype=dtype))
        self.init_fn = init_fn
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.init_fn is not None:
            self.init_fn(self)
        else:
            _default_embed_init(self.weight, self.pad_idx)

    def forward(self, x: Tensor) -> Tensor:
        return F.embedding(x, self.weight, self.pad_idx)

    def extra_repr(self) -> str:
        return f"num_embeddings={self.num_embeddings}, embed_dim={self.embed_dim}, pad_idx={self.pad_idx}"


class VocabShardedEmbedding(Embedding):
    """Rows (vocabulary) split over ``gang``: ids outside the local range embed
    to zero and the partial results are summed over the gang."""

    def __init__(self, gang: Gang, num_embeddings: int, embed_dim: int, pad_idx: int | None = None, *,
                 sequence_parallel: bool = False, init_fn: Callable[[StandardEmbedding], None] | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        """``sequence_parallel``: the output is this rank's shard of the tokens (``[T / W, D]``), i.e. the partial
        look-ups are reduce-scattered over the tokens instead of all-reduced."""
        super().__init__(num_embeddings, embed_dim, pad_idx)
        if num_embeddings % gang.size:
            raise ValueError(
                f"`num_embeddings` must be a multiple of `gang.size` ({gang.size}), but is {num_embeddings} instead.")
        self.gang = gang
        self.sequence_parallel = sequence_parallel
        self.sharded_num_embeddings = num_embeddings // gang.size
        self.weight = Parameter(torch.empty((self.sharded_num_embeddings, embed_dim), device=device, dtype=dtype))
        self.init_fn = init_fn
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.weight.device.type == "meta":
            return
        full = StandardEmbedding(self.num_embeddings, self.embed_dim, self.pad_idx, init_fn=self.init_fn,
                                 device=self.weight.device, dtype=self.weight.dtype)
        c = self.sharded_num_embeddings
        with torch.no_grad():
            self.weight.copy_(full.weight[self.gang.rank * c:(self.gang.rank + 1) * c])

    @staticmethod
    def from_embedding(embed: StandardEmbedding, gang: Gang) -> "VocabShardedEmbedding":
        m = VocabShardedEmbedding(gang, embed.num_embeddings, embed.embed_dim, embed.pad_idx, init_fn=embed.init_fn,
                                  device=torch.device("meta"), dtype=embed.weight.dtype)
        m.to_empty(device=embed.weight.device)
        c = m.sharded_num_embeddings
        with torch.no_grad():
            m.weight.copy_(embed.weight[gang.rank * c:(gang.rank + 1) * c])
        return m

    def forward(self, x: Tensor) -> Tensor:
        from fairseq2_b200.ops.embedding import embed_vocab_parallel

        lo = self.gang.rank * self.sharded_num_embeddings
        if self.sequence_parallel and self.gang.size > 1:
            from fairseq2_b200.ops.embedding import embed_vocab_parallel_scatter

            return embed_vocab_parallel_scatter(x, self.weight, lo, self.gang)
        y = embed_vocab_parallel(x, self.weight, lo)
        return reduce(y, self.gang)

    def to_embedding(self, device: Device | None = None) -> StandardEmbedding:
        w = gather(self.weight.detach(), self.gang, dim=0)
        e = StandardEmbedding(self.num_embeddings, self.embed_dim, self.pad_idx, device=torch.device("meta"),
                              dtype=self.weight.dtype)
        e.to_empty(device=device or self.weight.device)
        with torch.no_grad():
            e.weight.copy_(w)
        return e

    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        return [(self.weight, 0)]

    def extra_repr(self) -> str:
        return (f"tp_rank={self.gang.rank}, tp_size={self.gang.size}, num_embeddings={self.num_embeddings}, "
                f"sharded_num_embeddings={self.sharded_num_embeddings}, embed_dim={self.embed_dim}")


class ShardedEmbedding(Embedding):
    """Columns (embedding dimension) split over ``gang``; outputs are all-gathered."""

    def __init__(self, gang: Gang, num_embeddings: int, embed_dim: int, pad_idx: int | None = None, *,
                 init_fn: Callable[[StandardEmbedding], None] | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(num_embeddings, embed_dim, pad_idx)
        if embed_dim % gang.size:
            raise ValueError(f"`embed_dim` must be a multiple of `gang.size` ({gang.size}), but is {embed_dim} instead.")
        self.gang = gang
        self.sharded_embed_dim = embed_dim // gang.size
        self.weight = Parameter(torch.empty((num_embeddings, self.sharded_embed_dim), device=device, dtype=dtype))
        self.init_fn = init_fn
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.weight.device.type == "meta":
            return
        full = StandardEmbedding(self.num_embeddings, self.embed_dim, self.pad_idx, init_fn=self.init_fn,
                                 device=self.weight.device, dtype=self.weight.dtype)
        c = self.sharded_embed_dim
        with torch.no_grad():
            self.weight.copy_(full.weight[:, self.gang.rank * c:(self.gang.rank + 1) * c])

    @staticmethod
    def from_embedding(embed: StandardEmbedding, gang: Gang) -> "ShardedEmbedding":
        m = ShardedEmbedding(gang, embed.num_embeddings, embed.embed_dim, embed.pad_idx, init_fn=embed.init_fn,
                             device=torch.device("meta"), dtype=embed.weight.dtype)
        m.to_empty(device=embed.weight.device)
        c = m.sharded_embed_dim
        with torch.no_grad():
            m.weight.copy_(embed.weight[:, gang.rank * c:(gang.rank + 1) * c])
        return m

    def forward(self, x: Tensor) -> Tensor:
        y = F.embedding(x, self.weight, self.pad_idx)
        return gather(y, self.gang, dim=-1)

    def to_embedding(self, device: Device | None = None) -> StandardEmbedding:
        w = gather(self.weight.detach(), self.gang, dim=1)
        e = StandardEmbedding(self.num_embeddings, self.embed_dim, self.pad_idx, device=torch.device("meta"),
                              dtype=self.weight.dtype)
        e.to_empty(device=device or self.weight.device)
        with torch.no_grad():
            e.weight.copy_(w)
        return e

    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        return [(self.weight, 1)]


def init_scaled_embedding(embed: StandardEmbedding) -> None:
    """Normal(0, embed_dim^-0.5) with a zeroed pad row."""
    torch.nn.init.normal_(embed.weight, std=embed.embed_dim ** -0.5)
    if embed.pad_idx is not None:
        with torch.no_grad():
            embed.weight[embed.pad_idx].fill_(0.0)
