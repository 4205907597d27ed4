"""Model families (cf. fairseq2 ``models/family.py:72-808``,
``composition/models.py:183-247``).

A family bundles: config class + named archs, a factory, an optional
state-dict converter for foreign checkpoints (HF / reference keys), an FSDP
wrap policy, an activation-checkpointing applier and an HF exporter.
``create_new_model`` builds a randomly initialised model (optionally on the
meta device so that FSDP materialises it unit by unit); ``load_model``
downloads the checkpoint named by an asset card, streams it through the
delegating checkpoint loader with on-the-fly resharding to the current gangs,
and copies tensor by tensor into the model.
"""
from __future__ import annotations

from dataclasses import dataclass, field, is_dataclass, replace
from pathlib import Path
from typing import Any, Callable, Generic, Mapping, TypeVar

import torch
from torch.nn import Module

from fairseq2_b200.assets import AssetCard, AssetDownloadManager, AssetStore, get_asset_store
from fairseq2_b200.data_type import set_dtype
from fairseq2_b200.gang import Gangs, get_current_gangs, set_gangs
from fairseq2_b200.logging import log
from fairseq2_b200.model_checkpoint import ModelCheckpointLoader, create_default_checkpoint_loader
from fairseq2_b200.nn.sharded import get_shard_dims
from fairseq2_b200.nn.utils.module import broadcast_module
from fairseq2_b200.runtime.config_registry import ConfigNotFoundError, get_config_registry
from fairseq2_b200.typing import DataType, Device
from fairseq2_b200.utils.structured import StructureError, structure, unstructure
from fairseq2_b200.utils.config import merge_config

ModelT = TypeVar("ModelT", bound=Module)
ConfigT = TypeVar("ConfigT")


class ModelFamilyError(Exception):
    pass


class UnknownModelFamilyError(LookupError):
    pass


class UnknownModelArchitectureError(LookupError):
    pass


@dataclass
class ModelFamily(Generic[ModelT, ConfigT]):
    name: str
    kls: type
    config_kls: type
    factory: Callable[[Any], Module]
    state_dict_converter: Callable[[dict[str, Any], Any], dict[str, Any]] | None = None
    fsdp_wrap_policy: Callable[[Module], list[Module]] | None = None
    layerwise_ac_applier: Callable[[Module, int], None] | None = None
    hg_exporter: Callable[[Mapping[str, Any], Any], tuple[dict[str, Any], dict[str, Any]]] | None = None
    supports_meta: bool = True
    supports_fsdp: bool = True
    #: the factory builds every tensor-parallel layer (embedding, projections, output projection and loss) for
    #: token-sharded activations when ``parallel.tp.sequence_parallel()`` is active
    supports_sequence_parallel: bool = False
    restrict: bool = True

    # ------------------------------------------------------------------ config
    def get_archs(self) -> list[str]:
        return sorted(get_config_registry(self.config_kls).names())

    def get_arch_config(self, arch: str | None) -> Any:
        if arch is None:
            return self.config_kls()
        try:
            return get_config_registry(self.config_kls).get(arch)
        except ConfigNotFoundError:
            raise UnknownModelArchitectureError(
                f"'{arch}' is not a known architecture of the '{self.name}' model family.") from None

    def get_model_config(self, card: AssetCard, overrides: Mapping[str, Any] | None = None) -> Any:
        arch = card.maybe_get_field("model_arch", str)
        config = self.get_arch_config(arch)
        for key in ("model_config", "model_config_overrides"):
            o = card.maybe_get_field(key)
            if o:
                config = self.apply_config_overrides(config, o)
        if overrides:
            config = self.apply_config_overrides(config, overrides)
        return config

    def apply_config_overrides(self, config: Any, overrides: Mapping[str, Any]) -> Any:
        try:
            merged = merge_config(unstructure(config), dict(overrides))
            return structure(merged, self.config_kls)
        except (StructureError, TypeError) as ex:
            raise ModelFamilyError(f"The config overrides of the '{self.name}' family cannot be applied: {ex}") from ex

    # ------------------------------------------------------------------ create
    def create_new_model(self, config: Any, gangs: Gangs | None = None, dtype: DataType = torch.float32, *,
                         meta: bool = False, device: Device | None = None) -> Module:
        gangs = gangs or get_current_gangs()
        dev = torch.device("meta") if (meta and self.supports_meta) else (device or gangs.root.device)
        with dev, set_gangs(gangs, meta=True), set_dtype(dtype):
            model = self.factory(config)
        return model

    # -------------------------------------------------------------------- load
    def load_model(self, card: AssetCard | str, gangs: Gangs | None = None, dtype: DataType = torch.float32, *,
                   config: Any | None = None, config_overrides: Mapping[str, Any] | None = None, mmap: bool = False,
                   store: AssetStore | None = None, download_manager: AssetDownloadManager | None = None,
                   checkpoint_loader: ModelCheckpointLoader | None = None, strict: bool = True) -> Module:
        gangs = gangs or get_current_gangs()
        store = store or get_asset_store()
        if isinstance(card, str):
            card = store.retrieve_card(card)
        if config is None:
            config = self.get_model_config(card, config_overrides)
        uri = card.get_field("checkpoint", str)
        base = card.maybe_get_field("__base_path__", str)
        if base and "://" not in uri and not Path(uri).is_absolute():
            uri = str(Path(base) / uri)
        dm = download_manager or AssetDownloadManager()
        # rank 0 downloads first, the others then read the local copy
        if gangs.root.rank == 0:
            path = dm.download_model(uri, card.name)
        gangs.root.barrier()
        if gangs.root.rank != 0:
            path = dm.download_model(uri, card.name, local_only=True)
        sub = card.maybe_get_field("checkpoint_path", str)
        if sub:
            path = path / sub
        model = self.create_new_model(config, gangs, dtype)
        self.load_into(model, path, config, gangs, mmap=mmap, checkpoint_loader=checkpoint_loader, strict=strict,
                       restrict=card.maybe_get_field("restrict", bool) if card.has_field("restrict") else self.restrict)
        gangs.root.barrier()
        return model

    def load_into(self, model: Module, path: Path, config: Any, gangs: Gangs, *, mmap: bool = False,
                  checkpoint_loader: ModelCheckpointLoader | None = None, strict: bool = True,
                  restrict: bool = True) -> None:
        loader = checkpoint_loader or create_default_checkpoint_loader()
        shard_dims = get_shard_dims(model)
        conv = None
        if self.state_dict_converter is not None:
            fn = self.state_dict_converter

            def conv(sd: dict[str, Any]) -> dict[str, Any]:
                return fn(sd, config)

        state = dict(model.state_dict())
        seen: set[str] = set()
        # `model` holds whole (tensor-parallel-local) parameters at this point: the data-parallel engine shards them
        # later, unit by unit. The loader must therefore cut along the tensor-parallel dimension only.
        from fairseq2_b200.gang import FakeGang

        one = FakeGang(gangs.root.device)
        load_gangs = Gangs(root=gangs.root, dp=gangs.dp, rdp=gangs.rdp, sdp=one, tp=gangs.tp, pp=gangs.pp)
        with torch.no_grad():
            for key, tensor in loader.lazy_load(path, shard_dims, gangs=load_gangs, mmap=mmap, restrict=restrict,
                                                state_dict_converter=conv):
                tgt = state.get(key)
                if tgt is None:
                    if strict:
                        raise ModelFamilyError(f"The checkpoint has an unexpected key '{key}'.")
                    continue
                if tuple(tgt.shape) != tuple(tensor.shape):
                    raise ModelFamilyError(
                        f"The shape of '{key}' in the checkpoint is {tuple(tensor.shape)}, but {tuple(tgt.shape)} is expected.")
                tgt.copy_(tensor)
                seen.add(key)
        missing = [k for k in state if k not in seen]
        # tied parameters appear once in a checkpoint
        ptrs = {state[k].data_ptr() for k in seen}
        missing = [k for k in missing if state[k].data_ptr() not in ptrs]
        if strict and missing:
            raise ModelFamilyError(f"The checkpoint is missing the key(s) {missing}.")

    def iter_checkpoint(self, path: Path, config: Any, gangs: Gangs | None = None, **kw: Any):  # type: ignore[no-untyped-def]
        loader = create_default_checkpoint_loader()
        conv = None
        if self.state_dict_converter is not None:
            fn = self.state_dict_converter

            def conv(sd: dict[str, Any]) -> dict[str, Any]:
                return fn(sd, config)

        return loader.lazy_load(path, {}, gangs=gangs, state_dict_converter=conv, **kw)


_families: dict[str, ModelFamily[Any, Any]] = {}


def register_model_family(family: ModelFamily[Any, Any]) -> None:
    if family.name in _families:
        raise ValueError(f"The model family '{family.name}' is already registered.")
    _families[family.name] = family


def get_model_family(name: str) -> ModelFamily[Any, Any]:
    _ensure_builtin_families()
    try:
        return _families[name]
    except KeyError:
        raise UnknownModelFamilyError(f"'{name}' is not a known model family.") from None


def get_model_families() -> dict[str, ModelFamily[Any, Any]]:
    _ensure_builtin_families()
    return dict(_families)


_builtin_done = False


def _ensure_builtin_families() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from fairseq2_b200.models import registry  # noqa: F401  (registers every built-in family)
