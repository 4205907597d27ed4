"""Asset store (cf. fairseq2 ``assets/store.py:25-207``,
``metadata_provider.py:55-454``): cards come from metadata providers -- YAML
files shipped in the package, ``/etc/fairseq2/assets``,
``~/.config/fairseq2/assets``, extra directories, in-memory lists and
checkpoint directories. ``name@env`` variants overlay the base entry for the
detected environment; duplicate names across providers are an error."""
from __future__ import annotations

import os
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

from fairseq2_b200.assets.card import AssetCard, AssetCardError
from fairseq2_b200.utils.yaml import YamlError, load_yaml


class AssetMetadataError(Exception):
    pass


class AssetNotFoundError(LookupError):
    def __init__(self, name: str) -> None:
        super().__init__(f"An asset named '{name}' is not found.")
        self.name = name


class AssetMetadataProvider(ABC):
    @abstractmethod
    def load(self) -> dict[str, dict[str, Any]]:
        """``{"name[@env]": metadata}``"""


class InMemoryAssetMetadataProvider(AssetMetadataProvider):
    def __init__(self, entries: Sequence[Mapping[str, Any]], source: str = "memory") -> None:
        self._entries, self._source = list(entries), source

    def load(self) -> dict[str, dict[str, Any]]:
        out: dict[str, dict[str, Any]] = {}
        for e in self._entries:
            name = e.get("name")
            if not isinstance(name, str):
                raise AssetMetadataError(f"An asset entry of '{self._source}' does not have a valid 'name'.")
            if name in out:
                raise AssetMetadataError(f"'{self._source}' has more than one asset named '{name}'.")
            d = dict(e)
            d["__source__"] = self._source
            out[name] = d
        return out


class FileAssetMetadataProvider(AssetMetadataProvider):
    """Every ``*.yaml``/``*.yml`` under a directory; files may hold several documents."""

    def __init__(self, path: Path) -> None:
        self._path = path

    def load(self) -> dict[str, dict[str, Any]]:
        out: dict[str, dict[str, Any]] = {}
        if not self._path.exists():
            return out
        files = sorted(self._path.rglob("*.yaml")) + sorted(self._path.rglob("*.yml")) if self._path.is_dir() \
            else [self._path]
        for f in files:
            try:
                docs = load_yaml(f)
            except (YamlError, OSError) as ex:
                raise AssetMetadataError(f"The asset metadata file '{f}' cannot be loaded: {ex}") from ex
            for i, doc in enumerate(docs):
                if doc is None:
                    continue
                if not isinstance(doc, dict) or not isinstance(doc.get("name"), str):
                    raise AssetMetadataError(f"Document {i} of '{f}' must be a mapping with a 'name' key.")
                name = doc["name"]
                if name in out:
                    raise AssetMetadataError(f"Two assets under '{self._path}' have the same name '{name}'.")
                doc["__source__"] = str(f)
                doc["__base_path__"] = str(f.parent)
                out[name] = doc
        return out


def _detect_env() -> list[str]:
    envs = ["user"]
    e = os.environ.get("FAIRSEQ2_ASSET_ENV")
    if e:
        envs.append(e)
    return envs


class AssetStore:
    def __init__(self, providers: Sequence[AssetMetadataProvider] = (),
                 env_resolvers: Sequence[Callable[[], str | None]] = ()) -> None:
        self._providers = list(providers)
        self._env_resolvers = list(env_resolvers)
        self._cache: dict[str, dict[str, Any]] | None = None

    def add_provider(self, provider: AssetMetadataProvider, *, first: bool = False) -> None:
        if first:
            self._providers.insert(0, provider)
        else:
            self._providers.append(provider)
        self._cache = None

    def _all(self) -> dict[str, dict[str, Any]]:
        if self._cache is None:
            merged: dict[str, dict[str, Any]] = {}
            for p in self._providers:
                for name, md in p.load().items():
                    if name in merged:
                        raise AssetMetadataError(
                            f"Two assets have the same name '{name}' ({merged[name].get('__source__')} and {md.get('__source__')}).")
                    merged[name] = md
            self._cache = merged
        return self._cache

    def _envs(self) -> list[str]:
        envs = _detect_env()
        for r in self._env_resolvers:
            e = r()
            if e:
                envs.append(e)
        return envs

    def retrieve_card(self, name: str, *, envs: Sequence[str] | None = None, _chain: tuple[str, ...] = ()) -> AssetCard:
        if "@" in name:
            raise ValueError(f"`name` must not contain the reserved '@' character, but is '{name}' instead.")
        if name in _chain:
            raise AssetCardError(name, f"The asset cards {' -> '.join(_chain + (name,))} form a `base` cycle.")
        allmd = self._all()
        md = allmd.get(name) or allmd.get(name + "@")
        if md is None:
            raise AssetNotFoundError(name)
        md = dict(md)
        for env in (envs if envs is not None else self._envs()):
            over = allmd.get(f"{name}@{env}")
            if over is not None:
                md.update({k: v for k, v in over.items() if k != "name"})
                break
        md["name"] = name
        base = None
        base_name = md.get("base")
        if base_name is not None:
            if not isinstance(base_name, str):
                raise AssetCardError(name, f"The 'base' field of the '{name}' asset card must be a string.")
            base = self.retrieve_card(base_name, envs=envs, _chain=_chain + (name,))
        return AssetCard(name, md, base)

    def maybe_retrieve_card(self, name: str) -> AssetCard | None:
        try:
            return self.retrieve_card(name)
        except AssetNotFoundError:
            return None

    def retrieve_names(self) -> list[str]:
        return sorted({n.split("@")[0] for n in self._all()})


_default_store: AssetStore | None = None


def get_asset_dirs() -> list[Path]:
    dirs = [Path(__file__).parent / "cards"]
    sysd = Path(os.environ.get("FAIRSEQ2_ASSET_DIR", "/etc/fairseq2/assets"))
    if sysd.exists():
        dirs.append(sysd)
    userd = Path(os.environ.get("FAIRSEQ2_USER_ASSET_DIR", str(Path("~/.config/fairseq2/assets").expanduser())))
    if userd.exists():
        dirs.append(userd)
    return dirs


def get_asset_store() -> AssetStore:
    global _default_store
    if _default_store is None:
        _default_store = AssetStore([FileAssetMetadataProvider(d) for d in get_asset_dirs()])
    return _default_store


def register_checkpoint_models(store: AssetStore, checkpoint_dir: Path) -> None:
    """Exposes ``checkpoint_step_N`` / ``last_checkpoint`` / ``best_checkpoint`` cards of a checkpoint directory."""
    from fairseq2_b200.checkpoint.model_metadata import load_checkpoint_cards

    cards = load_checkpoint_cards(checkpoint_dir)
    if cards:
        store.add_provider(InMemoryAssetMetadataProvider(cards, source=str(checkpoint_dir)))
