"""Minimal URI value type (cf. ``src/fairseq2/utils/uri.py``)."""
from __future__ import annotations

import re
from pathlib import Path
from urllib.parse import urlparse

_SCHEME = re.compile(r"^[a-zA-Z][a-zA-Z0-9+.\-]*://")


class Uri:
    def __init__(self, s: str) -> None:
        if not _SCHEME.match(s):
            raise ValueError(f"'{s}' is not a URI.")
        self._s = s
        self._p = urlparse(s)

    @staticmethod
    def maybe_parse(s: str) -> "Uri | None":
        try:
            return Uri(s)
        except ValueError:
            return None

    @staticmethod
    def from_path(path: Path) -> "Uri":
        return Uri(path.expanduser().resolve().as_uri())

    @property
    def scheme(self) -> str:
        return self._p.scheme

    @property
    def netloc(self) -> str:
        return self._p.netloc

    @property
    def path(self) -> str:
        return self._p.path

    def to_path(self) -> Path:
        if self.scheme != "file":
            raise ValueError(f"Only file URIs can be converted to a path, but the scheme is '{self.scheme}'.")
        return Path(self._p.netloc + self._p.path)

    def __str__(self) -> str:
        return self._s

    def __repr__(self) -> str:
        return f"Uri('{self._s}')"

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Uri) and other._s == self._s

    def __hash__(self) -> int:
        return hash(self._s)
