"""YAML load/dump helpers over PyYAML (cf. ``src/fairseq2/utils/yaml.py``)."""
from __future__ import annotations

from pathlib import Path
from typing import IO, Any

import yaml


class YamlError(Exception):
    pass


def load_yaml(source: Path | IO[str] | str) -> list[Any]:
    """Loads every document of a (possibly multi-document) YAML source."""
    try:
        if isinstance(source, Path):
            with source.open("r", encoding="utf-8") as fp:
                return [d for d in yaml.safe_load_all(fp)]
        return [d for d in yaml.safe_load_all(source)]
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
