"""Asset cards (cf. fairseq2 ``assets/card.py:24-212``): named bundles of
metadata with ``base`` inheritance. Fields missing from a card fall through to
its base card."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

from fairseq2_b200.utils.structured import StructureError, structure


class AssetCardError(Exception):
    def __init__(self, name: str, message: str) -> None:
        super().__init__(message)
        self.name = name


class AssetCardFieldNotFoundError(AssetCardError):
    pass


class AssetCard:
    def __init__(self, name: str, metadata: Mapping[str, Any], base: "AssetCard | None" = None) -> None:
        self._name, self._metadata, self._base = name, dict(metadata), base

    @property
    def name(self) -> str:
        return self._name

    @property
    def metadata(self) -> Mapping[str, Any]:
        return self._metadata

    @property
    def base(self) -> "AssetCard | None":
        return self._base

    def has_field(self, name: str) -> bool:
        return name in self._metadata or (self._base is not None and self._base.has_field(name))

    def maybe_get_field(self, name: str, kls: Any = Any) -> Any:
        if name in self._metadata:
            v = self._metadata[name]
            if kls is Any:
                return v
            try:
                return structure(v, kls)
            except StructureError as ex:
                raise AssetCardError(self._name, f"The '{name}' field of the '{self._name}' asset card cannot be parsed as `{kls}`: {ex}") from ex
        if self._base is not None:
            return self._base.maybe_get_field(name, kls)
        return None

    def get_field(self, name: str, kls: Any = Any) -> Any:
        v = self.maybe_get_field(name, kls)
        if v is None and not self.has_field(name):
            raise AssetCardFieldNotFoundError(self._name, f"The '{self._name}' asset card does not have a field named '{name}'.")
        return v

    def field(self, name: str) -> "AssetCardField":
        return AssetCardField(self, name)

    def flatten(self) -> dict[str, Any]:
        out = self._base.flatten() if self._base is not None else {}
        out.update(self._metadata)
        return out

    def __repr__(self) -> str:
        return f"AssetCard(name={self._name!r}, metadata={self._metadata!r})"


class AssetCardField:
    def __init__(self, card: AssetCard, name: str) -> None:
        self._card, self._name = card, name

    def exists(self) -> bool:
        return self._card.has_field(self._name)

    def as_(self, kls: Any) -> Any:
        return self._card.get_field(self._name, kls)

    def as_uri_or_path(self) -> str:
        v = self._card.get_field(self._name, str)
        return v
