"""Dependency injection container (cf. fairseq2 ``runtime/dependency.py:38-470``).

``DependencyContainer.register(kls, factory, key=None, singleton=True)``
registers a provider; ``resolve(kls, key=None)`` builds (and for singletons
caches) the object; ``collection.register``/``resolve_all`` handle keyed
collections; ``register_type`` auto-wires a class from the type hints of its
``__init__``; cyclic resolutions are detected. A process-global resolver can be
swapped per recipe run (``set_dependency_resolver``)."""
from __future__ import annotations

import inspect
import threading
from typing import Any, Callable, Generic, Iterable, TypeVar, get_type_hints

T = TypeVar("T")


class DependencyError(Exception):
    pass


class DependencyNotFoundError(DependencyError):
    def __init__(self, kls: type, key: str | None) -> None:
        k = f" with key '{key}'" if key is not None else ""
        super().__init__(f"No provider is registered for `{getattr(kls, '__name__', kls)}`{k}.")
        self.kls, self.key = kls, key


class DependencyResolver:
    def resolve(self, kls: type[T], *, key: str | None = None) -> T:
        raise NotImplementedError

    def resolve_optional(self, kls: type[T], *, key: str | None = None) -> T | None:
        raise NotImplementedError

    def resolve_all(self, kls: type[T]) -> Iterable[tuple[str, T]]:
        raise NotImplementedError


Provider = Callable[[DependencyResolver], Any]


class DependencyContainer(DependencyResolver):
    def __init__(self) -> None:
        self._providers: dict[tuple[type, str | None], tuple[Provider, bool]] = {}
        self._instances: dict[tuple[type, str | None], Any] = {}
        self._resolving = threading.local()
        self._lock = threading.RLock()

    def register(self, kls: type[T], factory: Callable[[DependencyResolver], T], *, key: str | None = None,
                 singleton: bool = True) -> None:
        with self._lock:
            self._providers[(kls, key)] = (factory, singleton)
            self._instances.pop((kls, key), None)

    def register_instance(self, kls: type[T], obj: T, *, key: str | None = None) -> None:
        with self._lock:
            self._providers[(kls, key)] = (lambda r: obj, True)
            self._instances[(kls, key)] = obj

    def register_type(self, kls: type[T], impl: type[T] | None = None, *, key: str | None = None,
                      singleton: bool = True) -> None:
        impl = impl or kls

        def factory(resolver: DependencyResolver) -> T:
            return wire_object(resolver, impl)  # type: ignore[arg-type]

        self.register(kls, factory, key=key, singleton=singleton)

    def has(self, kls: type, *, key: str | None = None) -> bool:
        return (kls, key) in self._providers

    def resolve(self, kls: type[T], *, key: str | None = None) -> T:
        obj = self.resolve_optional(kls, key=key)
        if obj is None:
            raise DependencyNotFoundError(kls, key)
        return obj

    def resolve_optional(self, kls: type[T], *, key: str | None = None) -> T | None:
        k = (kls, key)
        with self._lock:
            if k in self._instances:
                return self._instances[k]  # type: ignore[no-any-return]
            entry = self._providers.get(k)
            if entry is None:
                return None
            stack = getattr(self._resolving, "stack", None)
            if stack is None:
                stack = self._resolving.stack = []
            if k in stack:
                chain = " -> ".join(getattr(c[0], "__name__", str(c[0])) for c in stack + [k])
                raise DependencyError(f"A cyclic dependency is detected: {chain}.")
            stack.append(k)
            try:
                factory, singleton = entry
                obj = factory(self)
            finally:
                stack.pop()
            if singleton and obj is not None:
                self._instances[k] = obj
            return obj  # type: ignore[no-any-return]

    def resolve_all(self, kls: type[T]) -> Iterable[tuple[str, T]]:
        for (c, key) in list(self._providers):
            if c is kls and key is not None:
                yield key, self.resolve(kls, key=key)


def wire_object(resolver: DependencyResolver, kls: type[T], **overrides: Any) -> T:
    """Instantiates ``kls`` resolving every ``__init__`` parameter by its type hint."""
    sig = inspect.signature(kls.__init__)
    try:
        hints = get_type_hints(kls.__init__)
    except Exception:  # noqa: BLE001
        hints = {}
    kwargs: dict[str, Any] = {}
    for name, p in list(sig.parameters.items())[1:]:
        if name in overrides:
            kwargs[name] = overrides[name]
            continue
        if p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        hint = hints.get(name)
        obj = resolver.resolve_optional(hint) if isinstance(hint, type) else None
        if obj is None:
            if p.default is not inspect.Parameter.empty:
                continue
            raise DependencyError(
                f"The parameter `{name}` of `{kls.__name__}` cannot be resolved (type hint: {hint}).")
        kwargs[name] = obj
    return kls(**kwargs)


_resolver: DependencyResolver | None = None


def get_dependency_resolver() -> DependencyResolver:
    global _resolver
    if _resolver is None:
        _resolver = DependencyContainer()
    return _resolver


def set_dependency_resolver(resolver: DependencyResolver | None) -> DependencyResolver | None:
    global _resolver
    old, _resolver = _resolver, resolver
    return old
