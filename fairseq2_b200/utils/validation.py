"""Recursive validation of config dataclasses (cf. ``src/fairseq2/utils/validation.py``).

Any object with ``validate() -> ValidationResult`` is ``Validatable``.
``ObjectValidator.validate(obj)`` walks dataclass fields, lists, dicts and
collects the errors of every nested validatable with a dotted field path.
"""
from __future__ import annotations

from dataclasses import fields, is_dataclass
from typing import Iterable, Protocol, runtime_checkable


class ValidationError(Exception):
    def __init__(self, result: "ValidationResult", field: str | None = None) -> None:
        lines = list(result.describe(field))
        super().__init__("\n".join(lines))
        self.result = result
        self.field = field


class ValidationResult:
    def __init__(self) -> None:
        self._errors: list[str] = []
        self._sub: dict[str, ValidationResult] = {}

    def add_error(self, message: str) -> None:
        self._errors.append(message)

    def add_sub_result(self, field: str, result: "ValidationResult") -> None:
        self._sub[field] = result

    @property
    def has_error(self) -> bool:
        return bool(self._errors) or any(r.has_error for r in self._sub.values())

    @property
    def errors(self) -> list[str]:
        return list(self._errors)

    def describe(self, field: str | None = None) -> Iterable[str]:
        prefix = field or "config"
        for e in self._errors:
            yield f"`{prefix}`: {e}"
        for name, sub in self._sub.items():
            if sub.has_error:
                yield from sub.describe(f"{field}.{name}" if field else name)


@runtime_checkable
class Validatable(Protocol):
    def validate(self) -> ValidationResult: ...


class ObjectValidator:
    def validate(self, obj: object) -> None:
        result = self._walk(obj)
        if result.has_error:
            raise ValidationError(result)

    def _walk(self, obj: object) -> ValidationResult:
        if isinstance(obj, Validatable) and not isinstance(obj, type):
            result = obj.validate()
            if not isinstance(result, ValidationResult):
                raise TypeError("`validate()` must return a `ValidationResult`.")
        else:
            result = ValidationResult()
        if is_dataclass(obj) and not isinstance(obj, type):
            for f in fields(obj):
                sub = self._walk(getattr(obj, f.name))
                if sub.has_error:
                    result.add_sub_result(f.name, sub)
        elif isinstance(obj, (list, tuple)):
            for i, e in enumerate(obj):
                sub = self._walk(e)
                if sub.has_error:
                    result.add_sub_result(f"[{i}]", sub)
        elif isinstance(obj, dict):
            for k, v in obj.items():
                sub = self._walk(v)
                if sub.has_error:
                    result.add_sub_result(str(k), sub)
        return result


def validate(obj: object) -> None:
    ObjectValidator().validate(obj)
