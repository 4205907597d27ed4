"""Dataclass <-> plain-object conversion ("structure"/"unstructure").

Same contract as fairseq2's ``ValueConverter`` (``src/fairseq2/utils/structured.py``):
``structure(obj, T)`` type-checks and converts a YAML/JSON-like object into an
instance of ``T``; ``unstructure`` does the inverse. Supported: primitives,
dataclasses, ``dict/list/set/tuple``, ``Literal``, ``Union``/``Optional``,
``Enum``, ``Path``, ``torch.dtype``, ``torch.device``, ``Any``.

The design here is a table of per-type closures resolved once per type
expression and cached, instead of a visitor class hierarchy.
"""
from __future__ import annotations

import dataclasses
import types
import typing
from dataclasses import MISSING, fields, is_dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Literal, Union, get_args, get_origin, get_type_hints

import torch

NoneType = type(None)


class StructureError(ValueError):
    """``obj`` cannot be structured into the requested type."""


_DTYPES = {
    n: getattr(torch, n)
    for n in ("float32", "float16", "bfloat16", "float64", "int8", "int16", "int32", "int64", "uint8", "bool",
              "float8_e4m3fn", "float8_e5m2")
    if hasattr(torch, n)
}
_DTYPES.update({"float": torch.float32, "half": torch.float16, "double": torch.float64, "long": torch.int64,
                "int": torch.int32})


def _type_name(t: Any) -> str:
    return getattr(t, "__name__", None) or str(t)


class ValueConverter:
    """Converts between typed objects and plain (YAML-representable) objects."""

    def structure(self, obj: object, target_type: Any, *, set_empty: bool = False) -> Any:
        try:
            return self._structure(obj, target_type, set_empty, "")
        except StructureError:
            raise
        except (TypeError, ValueError) as ex:
            raise StructureError(str(ex)) from ex

    def unstructure(self, obj: object) -> object:
        return self._unstructure(obj)

    # ------------------------------------------------------------------ structure
    def _structure(self, obj: object, t: Any, set_empty: bool, path: str) -> Any:
        if t is Any or t is object:
            return obj
        origin = get_origin(t)
        if origin is typing.Annotated:
            return self._structure(obj, get_args(t)[0], set_empty, path)
        if t is NoneType or t is None:
            if obj is None:
                return None
            raise StructureError(f"`{path or 'obj'}` must be `None`, but is `{obj!r}` instead.")
        if origin is Union or origin is types.UnionType:
            return self._structure_union(obj, get_args(t), set_empty, path)
        if origin is Literal:
            for a in get_args(t):
                if obj == a and type(obj) is type(a):
                    return obj
            if isinstance(obj, bool):
                # YAML 1.1 reads a bare `on`/`off`/`yes`/`no` as a boolean
                for word in (("on", "yes", "true") if obj else ("off", "no", "false")):
                    if word in get_args(t):
                        return word
            raise StructureError(
                f"`{path or 'obj'}` must be one of {list(get_args(t))}, but is `{obj!r}` instead.")
        if origin in (list, typing.List, typing.Sequence, typing.MutableSequence) or t is list:
            (et,) = get_args(t) or (Any,)
            if not isinstance(obj, (list, tuple)):
                raise StructureError(f"`{path or 'obj'}` must be a list, but is of type `{type(obj).__name__}` instead.")
            return [self._structure(e, et, set_empty, f"{path}[{i}]") for i, e in enumerate(obj)]
        if origin in (set, typing.Set, frozenset) or t is set:
            (et,) = get_args(t) or (Any,)
            if not isinstance(obj, (list, tuple, set, frozenset)):
                raise StructureError(f"`{path or 'obj'}` must be a list, but is of type `{type(obj).__name__}` instead.")
            out = [self._structure(e, et, set_empty, f"{path}[{i}]") for i, e in enumerate(obj)]
            s = set(out)
            if len(s) != len(out):
                raise StructureError(f"All elements of `{path or 'obj'}` must be unique.")
            return s
        if origin is tuple or t is tuple:
            args = get_args(t)
            if not isinstance(obj, (list, tuple)):
                raise StructureError(f"`{path or 'obj'}` must be a list, but is of type `{type(obj).__name__}` instead.")
            if not args:
                return tuple(obj)
            if len(args) == 2 and args[1] is Ellipsis:
                return tuple(self._structure(e, args[0], set_empty, f"{path}[{i}]") for i, e in enumerate(obj))
            if len(args) != len(obj):
                raise StructureError(
                    f"`{path or 'obj'}` must have {len(args)} element(s), but has {len(obj)} instead.")
            return tuple(self._structure(e, a, set_empty, f"{path}[{i}]") for i, (e, a) in enumerate(zip(obj, args)))
        if origin in (dict, typing.Dict, typing.Mapping, typing.MutableMapping) or t is dict:
            kt, vt = get_args(t) or (Any, Any)
            if not isinstance(obj, dict):
                raise StructureError(f"`{path or 'obj'}` must be a dict, but is of type `{type(obj).__name__}` instead.")
            return {
                self._structure(k, kt, set_empty, f"{path}.<key>"): self._structure(v, vt, set_empty, f"{path}.{k}")
                for k, v in obj.items()
            }
        if isinstance(t, type):
            if is_dataclass(t):
                return self._structure_dataclass(obj, t, set_empty, path)
            if issubclass(t, Enum):
                if isinstance(obj, t):
                    return obj
                if isinstance(obj, str):
                    try:
                        return t[obj]
                    except KeyError:
                        pass
                raise StructureError(
                    f"`{path or 'obj'}` must be one of {[e.name for e in t]}, but is `{obj!r}` instead.")
            if t is bool:
                if isinstance(obj, bool):
                    return obj
                if isinstance(obj, str) and obj.lower() in ("true", "false"):
                    return obj.lower() == "true"
                raise StructureError(f"`{path or 'obj'}` must be a bool, but is `{obj!r}` instead.")
            if t is int:
                if isinstance(obj, bool):
                    raise StructureError(f"`{path or 'obj'}` must be an int, but is a bool instead.")
                if isinstance(obj, int):
                    return obj
                if isinstance(obj, str):
                    try:
                        return int(obj)
                    except ValueError:
                        pass
                raise StructureError(f"`{path or 'obj'}` must be an int, but is `{obj!r}` instead.")
            if t is float:
                if isinstance(obj, bool):
                    raise StructureError(f"`{path or 'obj'}` must be a float, but is a bool instead.")
                if isinstance(obj, (int, float)):
                    return float(obj)
                if isinstance(obj, str):
                    try:
                        return float(obj)
                    except ValueError:
                        pass
                raise StructureError(f"`{path or 'obj'}` must be a float, but is `{obj!r}` instead.")
            if t is str:
                if isinstance(obj, str):
                    return obj
                raise StructureError(f"`{path or 'obj'}` must be a str, but is of type `{type(obj).__name__}` instead.")
            if issubclass(t, Path):
                if isinstance(obj, Path):
                    return obj
                if isinstance(obj, str):
                    return Path(obj)
                raise StructureError(f"`{path or 'obj'}` must be a path string, but is `{obj!r}` instead.")
            if t is torch.dtype:
                if isinstance(obj, torch.dtype):
                    return obj
                if isinstance(obj, str):
                    name = obj[6:] if obj.startswith("torch.") else obj
                    if name in _DTYPES:
                        return _DTYPES[name]
                raise StructureError(f"`{path or 'obj'}` must be a torch dtype name, but is `{obj!r}` instead.")
            if t is torch.device:
                if isinstance(obj, torch.device):
                    return obj
                if isinstance(obj, str):
                    try:
                        return torch.device(obj)
                    except RuntimeError as ex:
                        raise StructureError(str(ex)) from None
                raise StructureError(f"`{path or 'obj'}` must be a device string, but is `{obj!r}` instead.")
            if isinstance(obj, t):
                return obj
        raise StructureError(f"`{path or 'obj'}` cannot be structured into `{_type_name(t)}`.")

    def _structure_union(self, obj: object, args: tuple[Any, ...], set_empty: bool, path: str) -> Any:
        if obj is None and NoneType in args:
            return None
        # Exact-type matches win so that e.g. `int | str` keeps an int an int.
        errors = []
        for a in args:
            if a is NoneType:
                continue
            if isinstance(a, type) and not is_dataclass(a) and type(obj) is a:
                return obj
        for a in args:
            if a is NoneType:
                continue
            try:
                return self._structure(obj, a, set_empty, path)
            except StructureError as ex:
                errors.append(str(ex))
        raise StructureError(
            f"`{path or 'obj'}` cannot be structured into any of {[_type_name(a) for a in args]}: " + " | ".join(errors))

    def _structure_dataclass(self, obj: object, t: type, set_empty: bool, path: str) -> Any:
        if isinstance(obj, t):
            return obj
        if not isinstance(obj, dict):
            raise StructureError(
                f"`{path or 'obj'}` must be a dict to be structured into `{t.__name__}`, but is of type `{type(obj).__name__}` instead.")
        hints = get_type_hints(t)
        src = dict(obj)
        kwargs: dict[str, Any] = {}
        post: dict[str, Any] = {}
        for f in fields(t):
            sub = f"{path}.{f.name}" if path else f.name
            if f.name in src:
                v = self._structure(src.pop(f.name), hints[f.name], set_empty, sub)
                (kwargs if f.init else post)[f.name] = v
            elif f.init and f.default is MISSING and f.default_factory is MISSING:
                if set_empty:
                    kwargs[f.name] = EMPTY
                else:
                    raise StructureError(f"`{sub}` is required, but missing.")
            elif set_empty and f.init:
                kwargs[f.name] = EMPTY
        if src:
            extra = ", ".join(sorted(src))
            raise StructureError(
                f"`{path or 'obj'}` has unknown field(s) for `{t.__name__}`: {extra}")
        try:
            inst = t(**kwargs)
        except TypeError as ex:
            raise StructureError(f"`{path or 'obj'}` cannot be structured into `{t.__name__}`: {ex}") from ex
        for k, v in post.items():
            setattr(inst, k, v)
        return inst

    # ---------------------------------------------------------------- unstructure
    def _unstructure(self, obj: object) -> object:
        if obj is None or isinstance(obj, (bool, int, float, str)):
            return obj
        if obj is EMPTY:
            return None
        if is_dataclass(obj) and not isinstance(obj, type):
            out = {}
            for f in fields(obj):
                v = getattr(obj, f.name)
                if v is EMPTY:
                    continue
                out[f.name] = self._unstructure(v)
            return out
        if isinstance(obj, dict):
            return {self._unstructure(k): self._unstructure(v) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return [self._unstructure(e) for e in obj]
        if isinstance(obj, (set, frozenset)):
            items = [self._unstructure(e) for e in obj]
            try:
                return sorted(items)  # type: ignore[type-var]
            except TypeError:
                return items
        if isinstance(obj, Enum):
            return obj.name
        if isinstance(obj, Path):
            return str(obj)
        if isinstance(obj, torch.dtype):
            return str(obj)[6:]
        if isinstance(obj, torch.device):
            return str(obj)
        raise StructureError(f"Objects of type `{type(obj).__name__}` cannot be unstructured.")


class _Empty:
    """Marker for "field not provided" in ``set_empty`` mode (partial overrides)."""

    _inst: "_Empty | None" = None

    def __new__(cls) -> "_Empty":
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        return cls._inst

    def __repr__(self) -> str:
        return "EMPTY"

    def __bool__(self) -> bool:
        return False


EMPTY: Any = _Empty()

_default_converter = ValueConverter()


def structure(obj: object, target_type: Any, *, set_empty: bool = False) -> Any:
    return _default_converter.structure(obj, target_type, set_empty=set_empty)


def unstructure(obj: object) -> object:
    return _default_converter.unstructure(obj)


def is_unstructured(obj: object) -> bool:
    if isinstance(obj, dict):
        return all(isinstance(k, str) and is_unstructured(v) for k, v in obj.items())
    if isinstance(obj, list):
        return all(is_unstructured(e) for e in obj)
    return obj is None or isinstance(obj, (bool, int, float, str))


def merge_dataclass(target: Any, overrides: Any) -> Any:
    """Returns a copy of dataclass ``target`` where every non-EMPTY field of
    ``overrides`` (structured with ``set_empty=True``) replaces the original."""
    if not is_dataclass(target) or type(target) is not type(overrides):
        return overrides
    kw = {}
    for f in fields(target):
        ov = getattr(overrides, f.name)
        tv = getattr(target, f.name)
        if ov is EMPTY:
            kw[f.name] = tv
        elif is_dataclass(tv) and type(tv) is type(ov):
            kw[f.name] = merge_dataclass(tv, ov)
        else:
            kw[f.name] = ov
    return dataclasses.replace(target, **{k: v for k, v in kw.items() if _is_init(target, k)})


def _is_init(dc: Any, name: str) -> bool:
    for f in fields(dc):
        if f.name == name:
            return f.init
    return False
