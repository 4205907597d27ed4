"""Pattern-driven tensor-parallel sharding of an already built model.

The model factories of this package build sharded modules directly when ``gangs.tp.size > 1``; this module is
the older entry point kept for user models that are built unsharded: a mapping ``{regex over module paths ->
ShardSpec}`` selects ``Linear`` / ``StandardEmbedding`` children, which are replaced in place by their column-/row-
or vocabulary-/embedding-sharded counterparts (fairseq2 ``sharder.py:64-202``; deprecated upstream in favour of
sharding-aware modules, as here).
"""

from __future__ import annotations

import re
from abc import ABC, abstractmethod
from collections.abc import Iterable, Mapping
from dataclasses import dataclass

from torch.nn import Module

from fairseq2_b200.gang import Gangs
from fairseq2_b200.nn.embedding import ShardedEmbedding, StandardEmbedding, VocabShardedEmbedding
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, RowShardedLinear
from fairseq2_b200.utils.warn import warn_deprecated


@dataclass
class ShardSpec:
    dim: int
    """The sharded dimension of the weight."""

    region_boundary: bool = False
    """True when the sharded dimension borders another model-parallel region, so the gather (column) or scatter
    (row) at that border can be skipped."""


class ShardSpecError(Exception):
    pass


class ModuleSharder(ABC):
    @abstractmethod
    def shard(self, module: Module, gangs: Gangs, spec: ShardSpec) -> Module: ...

    @property
    @abstractmethod
    def supported_module_kls(self) -> type[Module]: ...


class LinearSharder(ModuleSharder):
    def shard(self, module: Module, gangs: Gangs, spec: ShardSpec) -> Module:
        if not isinstance(module, Linear):
            raise TypeError(f"`module` must be of type `{Linear}`, but is of type `{type(module)}` instead.")
        if spec.dim == 0:
            return ColumnShardedLinear.from_linear(module, gangs.tp, gather_output=not spec.region_boundary)
        if spec.dim == 1:
            return RowShardedLinear.from_linear(module, gangs.tp, scatter_input=not spec.region_boundary)
        raise ShardSpecError(f"`spec.dim` must be 0 or 1, but is {spec.dim} instead.")

    @property
    def supported_module_kls(self) -> type[Module]:
        return Linear


class EmbeddingSharder(ModuleSharder):
    def shard(self, module: Module, gangs: Gangs, spec: ShardSpec) -> Module:
        if not isinstance(module, StandardEmbedding):
            raise TypeError(f"`module` must be of type `{StandardEmbedding}`, but is of type `{type(module)}` instead.")
        if spec.region_boundary:
            raise ShardSpecError("`spec.region_boundary` must be `False`.")
        if spec.dim == 0:
            return VocabShardedEmbedding.from_embedding(module, gangs.tp)
        if spec.dim == 1:
            return ShardedEmbedding.from_embedding(module, gangs.tp)
        raise ShardSpecError(f"`spec.dim` must be 0 or 1, but is {spec.dim} instead.")

    @property
    def supported_module_kls(self) -> type[Module]:
        return StandardEmbedding


class ModelSharder(ABC):
    @abstractmethod
    def shard(self, model: Module, gangs: Gangs, specs: Mapping[str, ShardSpec]) -> None: ...


class StandardModelSharder(ModelSharder):
    def __init__(self, sharders: Iterable[ModuleSharder] | None = None) -> None:
        if sharders is None:
            sharders = (LinearSharder(), EmbeddingSharder())
        self._sharders = {s.supported_module_kls: s for s in sharders}

    def shard(self, model: Module, gangs: Gangs, specs: Mapping[str, ShardSpec]) -> None:
        warn_deprecated("Pattern-driven sharding is deprecated; build the model with `gangs` instead.")
        if gangs.tp.size == 1:
            return
        compiled = [(re.compile(pattern), pattern, spec) for pattern, spec in specs.items()]
        self._visit(model, gangs, compiled, "")

    def _visit(self, module: Module, gangs: Gangs, specs: list[tuple[re.Pattern[str], str, ShardSpec]], prefix: str) -> None:
        for name, child in list(module.named_children()):
            path = f"{prefix}.{name}" if prefix else name
            hit = next(((pattern, spec) for rx, pattern, spec in specs if rx.match(path)), None)
            if hit is None:
                self._visit(child, gangs, specs, path)
                continue
            pattern, spec = hit
            sharder = self._sharders.get(type(child))
            if sharder is None:
                raise ShardSpecError(f"The module at {path} matched by `specs['{pattern}']` is not shardable.")
            try:
                replacement = sharder.shard(child, gangs, spec)
            except ShardSpecError as ex:
                raise ShardSpecError(f"The shard specification of {path} matched by `specs['{pattern}']` is not valid. {ex}") from None
            module.register_module(name, replacement)
