"""YAML load/dump helpers over PyYAML (cf. ``src/fairseq2/utils/yaml.py``)."""
from __future__ import annotations

from pathlib import Path
from typing import IO, Any

import re

import yaml


class YamlError(Exception):
    pass


class _Loader(yaml.SafeLoader):
    """Safe loader that also reads ``1e-3`` / ``3E5`` (no dot) as floats, as YAML 1.2 does."""


_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(r"^[-+]?(?:[0-9][0-9_]*)(?:\.[0-9_]*)?[eE][-+]?[0-9]+$"),
    list("-+0123456789"))


def parse_yaml_value(text: str) -> Any:
    try:
        return yaml.load(text, Loader=_Loader)
    except yaml.YAMLError as ex:
        raise YamlError(f"The YAML value cannot be parsed: {ex}") from ex


def load_yaml(source: Path | IO[str] | str) -> list[Any]:
    """Loads every document of a (possibly multi-document) YAML source."""
    try:
        if isinstance(source, Path):
            with source.open("r", encoding="utf-8") as fp:
                return [d for d in yaml.load_all(fp, Loader=_Loader)]
        return [d for d in yaml.load_all(source, Loader=_Loader)]
    except yaml.YAMLError as ex:
        raise YamlError(f"The YAML source cannot be parsed: {ex}") from ex


def dump_yaml(obj: Any, target: Path | IO[str] | None = None) -> str | None:
    kw = dict(default_flow_style=False, sort_keys=False, allow_unicode=True)
    if target is None:
        return yaml.safe_dump(obj, **kw)
    if isinstance(target, Path):
        with target.open("w", encoding="utf-8") as fp:
            yaml.safe_dump(obj, fp, **kw)
        return None
    yaml.safe_dump(obj, target, **kw)
    return None


def read_yaml(path: Path) -> Any:
    docs = load_yaml(path)
    return docs[0] if docs else None
