"""Dataset families and hub (cf. fairseq2 ``datasets/family.py:31-190``, ``datasets/hub.py:33-335``).

A family binds a name to a dataset class, its config dataclass and an opener
``(name, config) -> dataset``. Datasets are opened from an asset card (fields
``dataset_family``, ``dataset_config``) or from an explicit family + config."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Generic, Mapping, TypeVar

from fairseq2_b200.assets import AssetCard, AssetNotFoundError, AssetStore, get_asset_store
from fairseq2_b200.utils.config import merge_config
from fairseq2_b200.utils.structured import StructureError, structure, unstructure

DatasetT = TypeVar("DatasetT")
ConfigT = TypeVar("ConfigT")


class UnknownDatasetFamilyError(LookupError):
    pass


class UnknownDatasetError(LookupError):
    pass


class DatasetError(Exception):
    pass


@dataclass
class DatasetFamily(Generic[DatasetT, ConfigT]):
    name: str
    kls: type
    config_kls: type
    opener: Callable[[str, Any], Any]

    def get_dataset_config(self, card: AssetCard | None, overrides: Mapping[str, Any] | Any | None = None) -> Any:
        cfg = unstructure(self.config_kls())
        if card is not None:
            c = card.maybe_get_field("dataset_config")
            if c:
                cfg = merge_config(cfg, c)
            base = card.maybe_get_field("__base_path__", str)
        if overrides is not None:
            if not isinstance(overrides, Mapping):
                overrides = unstructure(overrides)
            cfg = merge_config(cfg, dict(overrides))
        try:
            return structure(cfg, self.config_kls)
        except StructureError as ex:
            raise DatasetError(f"The configuration of the '{self.name}' dataset family is invalid: {ex}") from ex

    def open_dataset(self, name: str, config: Any) -> Any:
        return self.opener(name, config)


_FAMILIES: dict[str, DatasetFamily[Any, Any]] = {}


def register_dataset_family(name: str, kls: type, config_kls: type, opener: Callable[[str, Any], Any]) -> None:
    _FAMILIES[name] = DatasetFamily(name, kls, config_kls, opener)


def get_dataset_family(name: str) -> DatasetFamily[Any, Any]:
    try:
        return _FAMILIES[name]
    except KeyError:
        raise UnknownDatasetFamilyError(f"'{name}' is not a known dataset family; known: {sorted(_FAMILIES)}.") from None


def open_dataset(name: str | None = None, *, family: str | None = None, config_overrides: Any | None = None,
                 store: AssetStore | None = None, expected_kls: type | None = None) -> Any:
    """Opens a dataset by card name, or directly from ``family`` + ``config_overrides``."""
    card = None
    if name is not None:
        store = store or get_asset_store()
        try:
            card = store.retrieve_card(name)
        except AssetNotFoundError:
            if family is None:
                raise UnknownDatasetError(f"'{name}' is not a known dataset.") from None
        if card is not None:
            family = card.maybe_get_field("dataset_family", str) or family
    if family is None:
        raise UnknownDatasetFamilyError("The dataset family cannot be determined.")
    fam = get_dataset_family(family)
    config = fam.get_dataset_config(card, config_overrides)
    ds = fam.open_dataset(name or family, config)
    if expected_kls is not None and not isinstance(ds, expected_kls):
        raise TypeError(f"The dataset is expected to be a `{expected_kls.__name__}`, but is a `{type(ds).__name__}`.")
    return ds


class DatasetHub(Generic[DatasetT, ConfigT]):
    """Typed accessor of one family (``get_xxx_dataset_hub()`` in the reference)."""

    def __init__(self, family: str, store: AssetStore | None = None) -> None:
        self._family, self._store = family, store

    def iter_cards(self):  # type: ignore[no-untyped-def]
        store = self._store or get_asset_store()
        for n in store.retrieve_names():
            try:
                c = store.retrieve_card(n)
            except Exception:  # noqa: BLE001
                continue
            if c.maybe_get_field("dataset_family", str) == self._family:
                yield c

    def get_dataset_config(self, name: str) -> Any:
        store = self._store or get_asset_store()
        return get_dataset_family(self._family).get_dataset_config(store.retrieve_card(name))

    def open_dataset(self, name: str, config_overrides: Any | None = None) -> Any:
        return open_dataset(name, family=self._family, config_overrides=config_overrides, store=self._store)

    def open_custom_dataset(self, config: Any, name: str = "custom") -> Any:
        return get_dataset_family(self._family).open_dataset(name, config)
