"""Library composition and the extension mechanism (cf. fairseq2 ``composition/lib.py``, ``composition/extensions.py``)."""
from __future__ import annotations

import pytest

from fairseq2_b200.composition import ExtensionError, compose_library, register_tokenizer_family, run_extensions
from fairseq2_b200.composition.library import TokenizerFamily
from fairseq2_b200.utils.env import Environment
from fairseq2_b200.device import Device
from fairseq2_b200.file_system import FileSystem
from fairseq2_b200.models.family import ModelFamily
from fairseq2_b200.runtime.dependency import DependencyContainer
from fairseq2_b200.sharder import ModelSharder
from fairseq2_b200.world_info import WorldInfo


def _container(env: dict[str, str] | None = None) -> DependencyContainer:
    c = DependencyContainer()
    compose_library(c, env=env if env is not None else {"FAIRSEQ2_DEVICE": "cpu"})
    return c


def test_library_services_and_families() -> None:
    c = _container({"FAIRSEQ2_DEVICE": "cpu", "WORLD_SIZE": "4", "RANK": "3", "LOCAL_WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert c.resolve(Environment).get("RANK") == "3"
    w = c.resolve(WorldInfo)
    assert (w.rank, w.size, w.local_rank, w.local_size) == (3, 4, 1, 2)
    assert c.resolve(Device).type == "cpu"
    assert c.resolve(FileSystem) is c.resolve(FileSystem)            # singleton
    assert isinstance(c.resolve(ModelSharder), ModelSharder)
    families = dict(c.resolve_all(ModelFamily))
    for name in ("llama", "qwen", "mistral", "wav2vec2", "nllb"):
        assert name in families, name
    assert "llama3_8b" in families["llama"].get_archs()
    assert "char" in dict(c.resolve_all(TokenizerFamily))


class _Point:
    def __init__(self, value: str, fn) -> None:  # type: ignore[no-untyped-def]
        self.value, self._fn = value, fn

    def load(self):  # type: ignore[no-untyped-def]
        if isinstance(self._fn, Exception):
            raise self._fn
        return self._fn


def test_extensions_run_and_failures_are_contained(monkeypatch: pytest.MonkeyPatch) -> None:
    monkeypatch.delenv("FAIRSEQ2_EXTENSION_TRACE", raising=False)
    c = _container()
    seen: list[str] = []

    def good(container: DependencyContainer) -> None:
        seen.append("good")
        register_tokenizer_family(container, "test_composition_tok", lambda path, card: None)

    def bad(container: DependencyContainer) -> None:
        raise RuntimeError("boom")

    def wrong_signature() -> None:
        seen.append("never")

    ran = run_extensions(c, points=[_Point("pkg:good", good), _Point("pkg:bad", bad), _Point("pkg:wrong", wrong_signature),
                                    _Point("pkg:missing", ImportError("no module"))])
    assert ran == ["pkg:good"] and seen == ["good"]
    assert c.resolve(TokenizerFamily, key="test_composition_tok").name == "test_composition_tok"
    from fairseq2_b200.data.tokenizers import hub

    assert "test_composition_tok" in hub._families
    del hub._families["test_composition_tok"]


def test_extension_trace_raises(monkeypatch: pytest.MonkeyPatch) -> None:
    monkeypatch.setenv("FAIRSEQ2_EXTENSION_TRACE", "1")
    c = _container()

    def bad(container: DependencyContainer) -> None:
        raise RuntimeError("boom")

    with pytest.raises(ExtensionError) as info:
        run_extensions(c, points=[_Point("pkg:bad", bad)])
    assert info.value.entry_point == "pkg:bad" and isinstance(info.value.__cause__, RuntimeError)
    with pytest.raises(ExtensionError, match="signature"):
        run_extensions(c, points=[_Point("pkg:wrong", lambda: None)])


def test_init_is_idempotent_and_installs_the_resolver() -> None:
    import fairseq2_b200
    from fairseq2_b200.runtime.dependency import get_dependency_resolver, set_dependency_resolver

    calls: list[int] = []
    try:
        a = fairseq2_b200.init_fairseq2_b200(extras=lambda c: calls.append(1), no_extensions=True)
        b = fairseq2_b200.init_fairseq2_b200(extras=lambda c: calls.append(2), no_extensions=True)
        assert a is b and calls == [1]
        assert get_dependency_resolver() is a
    finally:
        fairseq2_b200._container = None
        set_dependency_resolver(None)


def test_asset_sources_added_through_the_container(tmp_path) -> None:  # type: ignore[no-untyped-def]
    from fairseq2_b200.assets import AssetStore
    from fairseq2_b200.composition import register_file_assets, register_in_memory_assets

    c = _container()
    c.register_instance(AssetStore, AssetStore([]))          # a private store: the process-wide one stays untouched
    (tmp_path / "cards.yaml").write_text("name: file_card\nmodel_family: llama\nmodel_arch: llama3_8b\n---\n"
                                         "name: file_card_b\nbase: file_card\n")
    register_file_assets(c, tmp_path)
    register_in_memory_assets(c, "test", [{"name": "mem_card", "tokenizer_family": "char"}])
    store = c.resolve(AssetStore)
    assert store.retrieve_card("file_card_b").maybe_get_field("model_arch", str) == "llama3_8b"
    assert store.retrieve_card("mem_card").maybe_get_field("tokenizer_family", str) == "char"
