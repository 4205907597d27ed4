"""Global model loading helpers (cf. fairseq2 ``models/hub.py:33-831``)."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Generic, Mapping, TypeVar

import torch
from torch.nn import Module

from fairseq2_b200.assets import AssetCard, AssetStore, get_asset_store
from fairseq2_b200.gang import Gangs
from fairseq2_b200.models.family import ModelFamily, UnknownModelFamilyError, get_model_family
from fairseq2_b200.typing import DataType

ModelT = TypeVar("ModelT", bound=Module)
ConfigT = TypeVar("ConfigT")


class ModelHub(Generic[ModelT, ConfigT]):
    """Typed accessor of one family: archs, configs, ``create_new_model``, ``load_model``."""

    def __init__(self, family: ModelFamily[Any, Any], store: AssetStore | None = None) -> None:
        self._family, self._store = family, store or get_asset_store()

    def get_archs(self) -> list[str]:
        return self._family.get_archs()

    def get_arch_config(self, arch: str) -> Any:
        return self._family.get_arch_config(arch)

    def get_model_config(self, card: AssetCard | str) -> Any:
        if isinstance(card, str):
            card = self._store.retrieve_card(card)
        return self._family.get_model_config(card)

    def create_new_model(self, config: Any, *, gangs: Gangs | None = None, dtype: DataType = torch.float32,
                         meta: bool = False) -> Module:
        return self._family.create_new_model(config, gangs, dtype, meta=meta)

    def load_model(self, card: AssetCard | str, *, gangs: Gangs | None = None, dtype: DataType = torch.float32,
                   config: Any | None = None, mmap: bool = False) -> Module:
        return self._family.load_model(card, gangs, dtype, config=config, mmap=mmap, store=self._store)

    def load_custom_model(self, path: Path, config: Any, *, gangs: Gangs | None = None,
                          dtype: DataType = torch.float32, mmap: bool = False, strict: bool = True) -> Module:
        from fairseq2_b200.gang import get_current_gangs

        gangs = gangs or get_current_gangs()
        model = self._family.create_new_model(config, gangs, dtype)
        self._family.load_into(model, path, config, gangs, mmap=mmap, strict=strict)
        return model


def get_model_hub(family_name: str) -> ModelHub[Any, Any]:
    return ModelHub(get_model_family(family_name))


# One accessor per built-in family, as in the reference (`get_llama_model_hub`, `get_qwen_model_hub`, ...:
# fairseq2 ``models/<family>/hub.py``).
def get_llama_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("llama")


def get_llama4_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("llama4")


def get_mistral_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("mistral")


def get_qwen_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("qwen")


def get_olmo_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("olmo")


def get_gemma3n_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("gemma3n")


def get_nllb_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("nllb")


def get_s2t_transformer_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("s2t_transformer")


def get_s2t_conformer_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("s2t_conformer")


def get_wav2vec2_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("wav2vec2")


def get_wav2vec2_asr_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("wav2vec2_asr")


def get_w2vbert_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("w2vbert")


def get_jepa_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("jepa")


def get_jepa_classifier_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("jepa_classifier")


def get_hg_model_hub() -> ModelHub[Any, Any]:
    return get_model_hub("hg")


def load_model(name_or_card: str | AssetCard, *, gangs: Gangs | None = None, dtype: DataType = torch.float32,
               config: Any | None = None, mmap: bool = False, store: AssetStore | None = None) -> Module:
    store = store or get_asset_store()
    card = store.retrieve_card(name_or_card) if isinstance(name_or_card, str) else name_or_card
    fam = card.maybe_get_field("model_family", str)
    if fam is None:
        raise UnknownModelFamilyError(f"The '{card.name}' asset card does not have a 'model_family' field.")
    return get_model_family(fam).load_model(card, gangs, dtype, config=config, mmap=mmap, store=store)
