"""Output sub-directory name derived from the configuration
(cf. fairseq2 ``recipe/internal/sweep_tag.py:46-219``): flatten the unstructured
config to ``path -> tag``, add ``world_size``, hash it, and safe-format
``sweep_format`` (unknown placeholders raise with the list of valid keys)."""
from __future__ import annotations

import hashlib
import re
import string
from typing import Any, Mapping


class SweepFormatError(ValueError):
    pass


class SweepFormatPlaceholderError(SweepFormatError):
    def __init__(self, unknown: list[str], valid: list[str]) -> None:
        super().__init__(f"`sweep_format` has unknown placeholder(s) {unknown}. Valid keys: {', '.join(valid[:50])}")
        self.unknown_keys = unknown


_SAFE = re.compile(r"[^-_\w]")


def _tag(v: Any) -> str:
    if v is None:
        return "none"
    if isinstance(v, bool):
        return "t" if v else "f"
    if isinstance(v, (int, float)):
        return f"{v}"
    s = _SAFE.sub("", str(v))
    if len(s) >= 16:
        return hashlib.sha1(str(v).encode()).hexdigest()[:8]
    return s


def _flatten(obj: Any, path: str, out: dict[str, str]) -> None:
    if isinstance(obj, Mapping):
        for k, v in obj.items():
            _flatten(v, f"{path}.{k}" if path else str(k), out)
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            _flatten(v, f"{path}[{i}]", out)
        out[path] = "-".join(_tag(v) for v in obj if not isinstance(v, (Mapping, list, tuple))) or "list"
    else:
        out[path] = _tag(obj)


def generate_sweep_tag(unstructured_config: Mapping[str, Any], world_size: int, sweep_format: str) -> str:
    tags: dict[str, str] = {}
    _flatten(unstructured_config, "", tags)
    tags["world_size"] = str(world_size)
    h = hashlib.sha1()
    for k in sorted(tags):
        h.update(f"{k}={tags[k]};".encode())
    tags["hash"] = h.hexdigest()[:8]
    try:
        fields = [f for _, f, _, _ in string.Formatter().parse(sweep_format) if f]
    except ValueError as ex:
        raise SweepFormatError(f"`sweep_format` must be a valid format string: {ex}") from None
    unknown = [f for f in fields if f not in tags]
    if unknown:
        raise SweepFormatPlaceholderError(unknown, sorted(tags))

    class _WholeKey(string.Formatter):
        """Looks a placeholder such as ``{model.name}`` or ``{list[0]}`` up as ONE key instead of walking attributes."""

        def get_field(self, field_name: str, args: Any, kwargs: Any) -> tuple[Any, str]:
            return kwargs[field_name], field_name

    out = _WholeKey().vformat(sweep_format, (), tags)
    return _SAFE.sub("", out.replace(".", "_DOT_")).replace("_DOT_", ".")
