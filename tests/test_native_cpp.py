"""Runs the C++ unit tests of the native data runtime (``csrc/data/tests/native_tests.cc``: tape, memory block, value
type, LRU file mapper, collater, converters and the pipeline operators with their record/reload/reset contracts) and
reports every case as one pytest case."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import pytest

_SO = Path(__file__).resolve().parent.parent / "fairseq2_b200" / "_data_tests.so"


def _rows():  # type: ignore[no-untyped-def]
    import torch  # noqa: F401  (the library links against libtorch)

    from fairseq2_b200.csrc.build import build_data_tests

    build_data_tests()   # a no-op unless a source is newer than the library
    name = "_data_tests"
    mod = sys.modules.get(name)
    if mod is None:
        spec = importlib.util.spec_from_file_location(name, _SO)
        assert spec is not None and spec.loader is not None
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return mod.run_all()


_ROWS = _rows()


def test_native_suite_is_not_empty() -> None:
    assert len(_ROWS) >= 25


@pytest.mark.parametrize("name,ok,message", _ROWS, ids=[r[0] for r in _ROWS])
def test_native_case(name: str, ok: bool, message: str) -> None:
    assert ok, f"{name}: {message}"
