"""Marker interface for modules that own a shard of a tensor-parallel parameter
(cf. fairseq2 ``nn/sharded.py:14-75``)."""
from __future__ import annotations

from typing import Protocol, runtime_checkable

from torch.nn import Module, Parameter


@runtime_checkable
class Sharded(Protocol):
    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        """(parameter, dimension along which it is sharded over the tp gang)."""


def get_shard_dims(module: Module) -> dict[str, int]:
    """Maps the fully-qualified name of every sharded parameter to its shard dim."""
    names = {id(p): n for n, p in module.named_parameters()}
    out: dict[str, int] = {}
    for m in module.modules():
        if isinstance(m, Sharded):
            for p, d in m.get_shard_dims():
                n = names.get(id(p))
                if n is not None:
                    out[n] = d
    return out
