"""Framework-wide exception types.

Mirrors the error taxonomy of fairseq2 (``src/fairseq2/error.py``): operational
failures (environment, I/O, network), internal invariants, invalid use,
unsupported features and malformed state dicts.
"""
from __future__ import annotations


class OperationalError(Exception):
    """A failure caused by the environment (disk, network, a peer rank)."""


class InternalError(Exception):
    """A broken internal invariant; always a bug in the framework."""


class InvalidOperationError(Exception):
    """The object is not in a state that allows the requested call."""


class NotSupportedError(Exception):
    """The requested feature is not available for this object."""


class StateDictError(Exception):
    """A state dict has missing, unexpected or malformed entries."""


class ContractError(Exception):
    """A user-supplied callback violated its documented contract."""


def raise_operational_system_error(cause: OSError) -> None:
    raise OperationalError("A system error occurred.") from cause
