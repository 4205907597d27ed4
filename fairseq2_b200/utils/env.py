"""Environment-variable access behind an interface so tests can fake it
(cf. ``src/fairseq2/utils/env.py``)."""
from __future__ import annotations

import os
from pathlib import Path
from typing import Iterator, Mapping, MutableMapping


class EnvironmentVariableError(Exception):
    def __init__(self, var_name: str, message: str) -> None:
        super().__init__(message)
        self.var_name = var_name


class Environment:
    def __init__(self, backing: MutableMapping[str, str] | None = None) -> None:
        self._m = os.environ if backing is None else backing

    def get(self, name: str) -> str:
        return self._m[name]

    def maybe_get(self, name: str, default: str | None = None) -> str | None:
        return self._m.get(name, default)

    def set(self, name: str, value: str) -> None:
        self._m[name] = value

    def has(self, name: str) -> bool:
        return name in self._m

    def to_dict(self) -> dict[str, str]:
        return dict(self._m)

    def __iter__(self) -> Iterator[str]:
        return iter(self._m)


def get_int(env: Mapping[str, str] | Environment, name: str, default: int | None = None) -> int | None:
    s = env.maybe_get(name) if isinstance(env, Environment) else env.get(name)
    if s is None:
        return default
    try:
        return int(s)
    except ValueError:
        raise EnvironmentVariableError(name, f"`{name}` must be an integer, but is '{s}' instead.") from None


def get_path(env: Mapping[str, str] | Environment, name: str) -> Path | None:
    s = env.maybe_get(name) if isinstance(env, Environment) else env.get(name)
    if not s:
        return None
    return Path(s).expanduser()


def get_rank(env: Mapping[str, str] | Environment) -> int:
    return get_int(env, "RANK", 0) or 0


def get_world_size(env: Mapping[str, str] | Environment) -> int:
    return get_int(env, "WORLD_SIZE", 1) or 1
