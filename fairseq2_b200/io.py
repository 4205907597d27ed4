"""Tensor file loading/dumping (cf. fairseq2 ``io.py:50-246``): ``torch.load``
with ``weights_only`` restriction and optional mmap, ``torch.save`` with a
chosen pickle protocol, and a safetensors loader."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from fairseq2_b200.typing import Device


class TensorFileError(Exception):
    def __init__(self, path: Path, message: str) -> None:
        super().__init__(message)
        self.path = path


class TensorFileLoader:
    def load(self, path: Path, *, map_location: Device | str | None = None, mmap: bool = False,
             restrict: bool = True) -> dict[str, Any]:
        try:
            return torch.load(path, map_location=map_location, weights_only=restrict, mmap=mmap or None)
        except FileNotFoundError:
            raise
        except (RuntimeError, OSError, EOFError, Exception) as ex:  # noqa: BLE001
            if isinstance(ex, FileNotFoundError):
                raise
            raise TensorFileError(path, f"The tensor file '{path}' cannot be loaded: {ex}") from ex


class TensorFileDumper:
    def dump(self, data: Mapping[str, Any], path: Path, *, pickle_protocol: int = 2) -> None:
        tmp = path.with_suffix(path.suffix + ".tmp")
        try:
            torch.save(dict(data), tmp, pickle_protocol=pickle_protocol)
            tmp.replace(path)
        except (RuntimeError, OSError) as ex:
            raise TensorFileError(path, f"The tensor file '{path}' cannot be saved: {ex}") from ex


class SafetensorsLoader:
    def load(self, path: Path, *, map_location: Device | str | None = None) -> dict[str, torch.Tensor]:
        try:
            from safetensors import safe_open
        except ImportError as ex:
            raise TensorFileError(path, "safetensors is not installed.") from ex
        files = sorted(path.glob("*.safetensors")) if path.is_dir() else [path]
        if not files:
            raise TensorFileError(path, f"No safetensors file found under '{path}'.")
        out: dict[str, torch.Tensor] = {}
        dev = str(map_location) if map_location is not None else "cpu"
        for f in files:
            try:
                with safe_open(f, framework="pt", device=dev) as fp:
                    for k in fp.keys():
                        if k in out:
                            raise TensorFileError(f, f"The key '{k}' exists in more than one safetensors file.")
                        out[k] = fp.get_tensor(k)
            except (RuntimeError, OSError) as ex:
                raise TensorFileError(f, f"The safetensors file '{f}' cannot be loaded: {ex}") from ex
        return out


def load_tensors(path: Path, **kw: Any) -> dict[str, Any]:
    return TensorFileLoader().load(path, **kw)


def dump_tensors(data: Mapping[str, Any], path: Path, **kw: Any) -> None:
    TensorFileDumper().dump(data, path, **kw)
