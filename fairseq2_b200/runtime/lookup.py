"""Read-only keyed views of one kind of object (cf. fairseq2 ``runtime/lookup.py:16-25``), e.g. all model families
registered in a container."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Generic, Hashable, Iterator, Mapping, TypeVar

from fairseq2_b200.runtime.dependency import DependencyResolver

T_co = TypeVar("T_co", covariant=True)


class Lookup(ABC, Generic[T_co]):
    @abstractmethod
    def maybe_get(self, key: Hashable) -> T_co | None: ...

    @abstractmethod
    def iter_keys(self) -> Iterator[Hashable]: ...

    @property
    @abstractmethod
    def kls(self) -> type[T_co]: ...

    def get(self, key: Hashable) -> T_co:
        obj = self.maybe_get(key)
        if obj is None:
            raise LookupError(f"No `{self.kls.__name__}` is registered under '{key}'.")
        return obj


class MappingLookup(Lookup[T_co]):
    def __init__(self, kls: type[T_co], items: Mapping[Hashable, T_co]) -> None:
        self._kls, self._items = kls, items

    def maybe_get(self, key: Hashable) -> T_co | None:
        return self._items.get(key)

    def iter_keys(self) -> Iterator[Hashable]:
        return iter(self._items)

    @property
    def kls(self) -> type[T_co]:
        return self._kls


class ResolverLookup(Lookup[T_co]):
    """The keyed registrations of ``kls`` in a dependency resolver."""

    def __init__(self, resolver: DependencyResolver, kls: type[T_co]) -> None:
        self._resolver, self._kls = resolver, kls

    def maybe_get(self, key: Hashable) -> T_co | None:
        return self._resolver.resolve_optional(self._kls, key=str(key))

    def iter_keys(self) -> Iterator[Hashable]:
        for key, _ in self._resolver.resolve_all(self._kls):
            yield key

    @property
    def kls(self) -> type[T_co]:
        return self._kls
