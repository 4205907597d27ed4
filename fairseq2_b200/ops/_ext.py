"""Loader of the in-tree native extension.

The extension is built by ``fairseq2_b200/csrc/build.py`` (nvcc, sm_100a only)
into ``fairseq2_b200/_C.so``; it is imported from that path and never from
site-packages.
"""
from __future__ import annotations

import importlib.util
import os
from contextlib import contextmanager
from typing import Iterator
import sys
from pathlib import Path
from types import ModuleType

_PKG_DIR = Path(__file__).resolve().parent.parent
_ext: ModuleType | None = None
_err: str | None = None


def _so_path(name: str) -> Path:
    return _PKG_DIR / f"{name}.so"


def _load(name: str) -> ModuleType:
    import torch  # noqa: F401  (the extension links against libtorch)

    path = _so_path(name)
    if not path.exists():
        raise ImportError(
            f"The native extension '{path}' has not been built. Run `python -m fairseq2_b200.csrc.build`.")
    spec = importlib.util.spec_from_file_location(f"fairseq2_b200.{name}", path)
    if spec is None or spec.loader is None:
        raise ImportError(f"'{path}' cannot be loaded as a Python extension module.")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[f"fairseq2_b200.{name}"] = mod
    spec.loader.exec_module(mod)
    return mod


def get_ext() -> ModuleType:
    """Returns the CUDA kernel extension; raises ``ImportError`` if it is not built."""
    global _ext, _err
    if _ext is None:
        if _err is not None:
            raise ImportError(_err)
        try:
            _ext = _load("_C")
        except ImportError as ex:
            _err = str(ex)
            raise
        _install_status_check(_ext)
    return _ext


class KernelWaitTimeout(RuntimeError):
    """A kernel gave up on a bounded wait (a peer never signalled, a copy never landed) and returned early."""

    def __init__(self, code: int, site: int) -> None:
        super().__init__(f"a fairseq2_b200 kernel gave up on a bounded wait (code {code}, site {site})")
        self.code, self.site = code, site


def _install_status_check(mod: ModuleType) -> None:
    """``ext.check_status()`` is evaluated in Python: it reads the host-mapped status word, clears it and raises
    ``KernelWaitTimeout``. The error therefore never travels through C++ unwinding of a process whose GPU peers may
    already be gone."""

    def check_status() -> None:
        status = int(mod.read_status())
        if status != 0:
            mod.reset_status()
            raise KernelWaitTimeout(status & 0xFF, status >> 8)

    mod.check_status = check_status  # type: ignore[attr-defined]


def ext_available() -> bool:
    try:
        get_ext()
        return True
    except ImportError:
        return False


def require_ext() -> ModuleType:
    """Used on CUDA paths: the kernels are mandatory there."""
    try:
        return get_ext()
    except ImportError as ex:
        raise RuntimeError(
            "A CUDA tensor reached a fairseq2_b200 op but the sm_100a kernel extension is not available: "
            f"{ex}") from ex


_kernels_on = True


@contextmanager
def kernels_enabled(value: bool) -> Iterator[None]:
    """Temporarily routes CUDA tensors through the PyTorch formulations (``value=False``); used by tests that
    compare a kernel path with its oracle on the same device."""
    global _kernels_on
    old, _kernels_on = _kernels_on, value
    try:
        yield
    finally:
        _kernels_on = old


def use_kernels(*tensors: object) -> bool:
    """True when the op must run on the native kernels (any CUDA tensor input)."""
    import torch

    for t in tensors:
        if isinstance(t, torch.Tensor) and t.is_cuda:
            if not _kernels_on or os.environ.get("FAIRSEQ2_B200_FORCE_TORCH") == "1":
                return False
            return True
    return False
