"""Registration of the toolkit's services and families in a ``DependencyContainer``.

Counterpart of the reference's ``_register_library`` (``fairseq2/composition/lib.py:119-260``) and of its
``register_model_family`` / ``register_dataset_family`` / ``register_tokenizer_family`` helpers
(``fairseq2/composition/models.py``, ``datasets.py``, ``tokenizers.py``). The helpers here write to BOTH the container
and the module registries that ``load_model`` / ``open_dataset`` / ``load_tokenizer`` consult, so a family added by an
extension is usable from recipes and from resolver-based code alike.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

import torch

from fairseq2_b200.assets import AssetDownloadManager, AssetStore, get_asset_store
from fairseq2_b200.assets.store import FileAssetMetadataProvider, InMemoryAssetMetadataProvider
from fairseq2_b200.cluster import ClusterHandler, SlurmHandler
from fairseq2_b200.datasets.family import DatasetFamily
from fairseq2_b200.datasets.family import register_dataset_family as _register_dataset_family_global
from fairseq2_b200.device import Device, detect_default_device
from fairseq2_b200.file_system import FileSystem, GlobalFileSystem
from fairseq2_b200.models.family import ModelFamily, get_model_families
from fairseq2_b200.models.family import register_model_family as _register_model_family_global
from fairseq2_b200.runtime.dependency import DependencyContainer, DependencyResolver
from fairseq2_b200.sharder import EmbeddingSharder, LinearSharder, ModelSharder, ModuleSharder, StandardModelSharder
from fairseq2_b200.utils.env import Environment
from fairseq2_b200.utils.rng import RngBag
from fairseq2_b200.utils.threading import StandardThreadPool, ThreadPool
from fairseq2_b200.world_info import WorldInfo


class TokenizerFamily:
    """A named tokenizer loader (the module registry keeps the bare callable)."""

    def __init__(self, name: str, loader: Callable[..., Any]) -> None:
        self.name, self.loader = name, loader


def register_model_family(container: DependencyContainer, family: ModelFamily[Any, Any]) -> None:
    _register_model_family_global(family)
    container.register_instance(ModelFamily, family, key=family.name)


def register_dataset_family(container: DependencyContainer, name: str, kls: type, config_kls: type,
                            opener: Callable[[str, Any], Any]) -> None:
    _register_dataset_family_global(name, kls, config_kls, opener)
    container.register_instance(DatasetFamily, DatasetFamily(name, kls, config_kls, opener), key=name)


def register_tokenizer_family(container: DependencyContainer, name: str, loader: Callable[..., Any]) -> None:
    from fairseq2_b200.data.tokenizers.hub import register_tokenizer_family as register_global

    register_global(name, loader)
    container.register_instance(TokenizerFamily, TokenizerFamily(name, loader), key=name)


# ------------------------------------------------------------------ asset sources
# cf. fairseq2 ``composition/assets.py:37-62``: each helper adds one source of asset cards to the store that the
# container hands out (and that ``load_model`` / ``load_tokenizer`` / ``open_dataset`` use by default).
def register_file_assets(container: DependencyContainer, path: Path) -> None:
    """All ``*.yaml`` cards under ``path`` (a file or a directory)."""
    container.resolve(AssetStore).add_provider(FileAssetMetadataProvider(Path(path)))


def register_package_assets(container: DependencyContainer, package: str) -> None:
    """The cards shipped inside an importable package, e.g. ``"my_extension.cards"``."""
    import importlib

    mod = importlib.import_module(package)
    paths = list(getattr(mod, "__path__", []))
    if not paths:
        raise ValueError(f"`package` must be an importable package with a directory, but '{package}' is not.")
    store = container.resolve(AssetStore)
    for p in paths:
        store.add_provider(FileAssetMetadataProvider(Path(p)))


def register_in_memory_assets(container: DependencyContainer, source: str,
                              entries: Sequence[Mapping[str, Any]]) -> None:
    container.resolve(AssetStore).add_provider(InMemoryAssetMetadataProvider(entries, source=source))


def register_checkpoint_models(container: DependencyContainer, checkpoint_dir: Path) -> None:
    """``checkpoint_step_N`` / ``last_checkpoint`` / ``best_checkpoint`` cards of a training run."""
    from fairseq2_b200.assets.store import register_checkpoint_models as register

    register(container.resolve(AssetStore), Path(checkpoint_dir))


def compose_library(container: DependencyContainer, *, env: Mapping[str, str] | None = None) -> None:
    """Registers the process-wide services and every built-in family."""
    # the process environment, or the mapping a test passes in
    environ = Environment(None if env is None else dict(env))
    container.register_instance(Environment, environ)

    container.register(WorldInfo, lambda r: WorldInfo.from_env(r.resolve(Environment).to_dict()))
    container.register(Device, lambda r: detect_default_device(r.resolve(Environment).to_dict()))
    container.register(FileSystem, lambda r: GlobalFileSystem())
    container.register(ThreadPool, lambda r: StandardThreadPool(max_num_workers=1, num_torch_threads=1))
    container.register(AssetStore, lambda r: get_asset_store())
    container.register(AssetDownloadManager, lambda r: AssetDownloadManager())

    def rng_bag(r: DependencyResolver) -> RngBag:
        device = r.resolve(Device)
        cpu = torch.device("cpu")
        return RngBag.from_device_defaults(cpu) if device.type == "cpu" else RngBag.from_device_defaults(cpu, device)

    container.register(RngBag, rng_bag)

    # sharders: a keyed collection that the model sharder consumes
    container.register(ModuleSharder, lambda r: LinearSharder(), key="linear")
    container.register(ModuleSharder, lambda r: EmbeddingSharder(), key="embedding")
    container.register(ModelSharder, lambda r: StandardModelSharder([s for _, s in r.resolve_all(ModuleSharder)]))
    container.register(ClusterHandler, lambda r: SlurmHandler(), key="slurm")

    # families: mirror the module registries (built-ins register themselves there on first use)
    for name, family in get_model_families().items():
        container.register_instance(ModelFamily, family, key=name)
    from fairseq2_b200.datasets import family as dataset_family_mod

    for name, fam in dataset_family_mod._FAMILIES.items():
        container.register_instance(DatasetFamily, fam, key=name)
    from fairseq2_b200.data.tokenizers import hub as tokenizer_hub

    for name, loader in tokenizer_hub._families.items():
        container.register_instance(TokenizerFamily, TokenizerFamily(name, loader), key=name)
