"""Config overlay merge and string directives (cf. ``src/fairseq2/utils/config.py``).

``merge(base, overrides)`` deep-merges mappings. Inside any mapping of the
overrides two control keys are honoured: ``_del_: [k, ...]`` removes keys of the
base mapping, ``_set_: {k: v}`` replaces keys wholesale (no deep merge).
Directives rewrite string leaves: ``${dir}`` -> directory of the config file,
``${env:NAME}`` / ``${env:NAME:default}`` -> environment variable.
"""
from __future__ import annotations

import os
import re
from copy import deepcopy
from pathlib import Path
from typing import Callable, Mapping, Sequence

Directive = Callable[[str], object]


def merge_config(base: object, overrides: object, _path: str = "") -> object:
    if not isinstance(overrides, Mapping):
        return deepcopy(overrides)
    tgt: Mapping[str, object] = base if isinstance(base, Mapping) else {}

    dels = overrides.get("_del_")
    if dels is not None and (not isinstance(dels, list) or not all(isinstance(k, str) for k in dels)):
        raise TypeError(f"`{_path}_del_` in the overrides must be a list of strings.")
    sets = overrides.get("_set_")
    if sets is not None and (not isinstance(sets, Mapping) or not all(isinstance(k, str) for k in sets)):
        raise TypeError(f"`{_path}_set_` in the overrides must be a mapping with string keys.")

    skip = set(dels or ())
    out = {k: deepcopy(v) for k, v in tgt.items() if k not in skip}
    for k, v in overrides.items():
        if k in ("_del_", "_set_"):
            continue
        if isinstance(v, Mapping):
            out[k] = merge_config(out.get(k), v, f"{_path}{k}.")
        else:
            out[k] = deepcopy(v)
    for k, v in (sets or {}).items():
        out[k] = deepcopy(v)
    return out


_ENV_RE = re.compile(r"\$\{env:([A-Za-z_][A-Za-z0-9_]*)(?::([^}]*))?\}")


def replace_env_directive(env: Mapping[str, str] | None = None) -> Directive:
    e = os.environ if env is None else env

    def run(s: str) -> object:
        return _ENV_RE.sub(lambda m: e.get(m.group(1), m.group(2) or ""), s)

    return run


def replace_path_directive(config_dir: Path) -> Directive:
    d = str(config_dir)

    def run(s: str) -> object:
        return s.replace("${dir}", d)

    return run


def process_directives(obj: object, directives: Sequence[Directive]) -> object:
    if not directives:
        return obj
    if isinstance(obj, list):
        return [process_directives(e, directives) for e in obj]
    if isinstance(obj, dict):
        return {k: process_directives(v, directives) for k, v in obj.items()}
    if isinstance(obj, str):
        cur: object = obj
        for d in directives:
            if not isinstance(cur, str):
                break
            cur = d(cur)
        return cur
    return obj


class ConfigMerger:
    """Object form of :func:`merge_config` for dependency injection."""

    def merge(self, unstructured_config: object, overrides: object) -> object:
        return merge_config(unstructured_config, overrides)


class ConfigProcessor:
    def __init__(self, default_directives: Sequence[Directive] = ()) -> None:
        self._defaults = list(default_directives)

    def process(self, unstructured_config: object, directives: Sequence[Directive] | None = None) -> object:
        return process_directives(unstructured_config, [*self._defaults, *(directives or [])])


def parse_config_overrides(pairs: Sequence[str]) -> dict[str, object]:
    """``["a.b=1", "c=[1,2]"]`` -> nested dict, values parsed as YAML scalars."""
    from fairseq2_b200.utils.yaml import YamlError, parse_yaml_value

    out: dict[str, object] = {}
    for item in pairs:
        if "=" not in item:
            raise ValueError(f"A config override must be of the form key=value, but is '{item}' instead.")
        key, raw = item.split("=", 1)
        try:
            val = parse_yaml_value(raw)
        except YamlError as ex:
            raise ValueError(f"The value of '{key}' is not valid YAML: {ex}") from None
        cur = out
        parts = key.strip().split(".")
        if not all(parts):
            raise ValueError(f"'{key}' is not a valid config key.")
        for p in parts[:-1]:
            nxt = cur.setdefault(p, {})
            if not isinstance(nxt, dict):
                raise ValueError(f"'{key}' conflicts with an earlier override.")
            cur = nxt
        cur[parts[-1]] = val
    return out
