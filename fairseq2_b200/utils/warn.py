"""Deprecation-warning switches (fairseq2 ``utils/warn.py:12-33``)."""

from __future__ import annotations

import warnings


def enable_deprecation_warnings() -> None:
    """Show each ``DeprecationWarning`` raised from this package once. Recipe entry points call this."""
    warnings.filterwarnings("once", category=DeprecationWarning, module=r"fairseq2_b200\..*")


def warn_deprecated(msg: str) -> None:
    warnings.warn(msg, DeprecationWarning, stacklevel=3)
