"""Named configuration presets ("architectures") per config class
(cf. fairseq2 ``runtime/config_registry.py:49-110``).

``registry = ConfigRegistry(LLaMAConfig)``; ``@registry.decorator("llama3_8b")``
registers a zero-argument factory; ``registry.get("llama3_8b")`` builds a fresh
config each time so callers may mutate the result.
"""
from __future__ import annotations

from typing import Callable, Generic, Iterable, TypeVar

ConfigT = TypeVar("ConfigT")


class ConfigNotFoundError(LookupError):
    def __init__(self, name: str) -> None:
        super().__init__(f"A configuration named '{name}' is not registered.")
        self.name = name


class ConfigRegistry(Generic[ConfigT]):
    def __init__(self, config_kls: type[ConfigT]) -> None:
        self.config_kls = config_kls
        self._factories: dict[str, Callable[[], ConfigT]] = {}

    def register(self, name: str, factory: Callable[[], ConfigT]) -> None:
        if name in self._factories:
            raise ValueError(f"`name` must be unique, but '{name}' is already registered.")
        self._factories[name] = factory

    def decorator(self, name: str) -> Callable[[Callable[[], ConfigT]], Callable[[], ConfigT]]:
        def wrap(fn: Callable[[], ConfigT]) -> Callable[[], ConfigT]:
            self.register(name, fn)
            return fn

        return wrap

    def get(self, name: str) -> ConfigT:
        try:
            return self._factories[name]()
        except KeyError:
            raise ConfigNotFoundError(name) from None

    def names(self) -> Iterable[str]:
        return self._factories.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._factories


_registries: dict[type, ConfigRegistry] = {}  # type: ignore[type-arg]


def get_config_registry(config_kls: type[ConfigT]) -> ConfigRegistry[ConfigT]:
    r = _registries.get(config_kls)
    if r is None:
        r = _registries[config_kls] = ConfigRegistry(config_kls)
    return r


class ConfigRegistrar(Generic[ConfigT]):
    """``arch = ConfigRegistrar(LLaMAConfig)``; ``@arch("name")`` registers a preset."""

    def __init__(self, config_kls: type[ConfigT]) -> None:
        self._registry = get_config_registry(config_kls)

    def __call__(self, name: str) -> Callable[[Callable[[], ConfigT]], Callable[[], ConfigT]]:
        return self._registry.decorator(name)
