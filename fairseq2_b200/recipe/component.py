"""Named, configurable components (optimizers, LR schedulers, samplers, ...)
resolved from ``{name, config}`` sections (cf. fairseq2 ``recipe/component.py:44-109``)."""
from __future__ import annotations

from typing import Any, Callable, Mapping

from fairseq2_b200.utils.structured import StructureError, structure


class UnknownComponentError(LookupError):
    def __init__(self, kind: str, name: str, known: list[str]) -> None:
        super().__init__(f"'{name}' is not a known {kind}. Known {kind}s: {', '.join(sorted(known))}.")
        self.kind, self.name = kind, name


_registry: dict[str, dict[str, tuple[type | None, Callable[..., Any]]]] = {}


def register_component(kind: str, name: str, config_kls: type | None, factory: Callable[..., Any]) -> None:
    _registry.setdefault(kind, {})[name] = (config_kls, factory)


def create_component(kind: str, name: str, config: Mapping[str, Any] | None, *args: Any, **kw: Any) -> Any:
    table = _registry.get(kind, {})
    entry = table.get(name)
    if entry is None:
        raise UnknownComponentError(kind, name, list(table))
    config_kls, factory = entry
    cfg: Any = config or {}
    if config_kls is not None:
        try:
            cfg = structure(dict(cfg), config_kls)
        except StructureError as ex:
            raise ValueError(f"The configuration of the '{name}' {kind} is invalid: {ex}") from ex
    return factory(cfg, *args, **kw)


def component_names(kind: str) -> list[str]:
    return sorted(_registry.get(kind, {}))
