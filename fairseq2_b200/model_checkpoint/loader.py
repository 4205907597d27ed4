"""Model checkpoint loaders (cf. fairseq2 ``model_checkpoint/*``): a delegating
loader over {native rank-sharded directory, ``.pt/.pth/.bin`` files,
safetensors, LLaMA ``consolidated.NN.pth``}. Every loader yields
``(key, tensor)`` lazily, already resharded for the caller's gangs and with an
optional key/layout converter applied."""
from __future__ import annotations

import re
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Callable, Iterator, Mapping

import torch
from torch import Tensor

from fairseq2_b200.gang import Gangs
from fairseq2_b200.io import SafetensorsLoader, TensorFileError, TensorFileLoader
from fairseq2_b200.model_checkpoint.common import reshard_tensor

StateDictConverter = Callable[[dict[str, object]], dict[str, object]]


class ModelCheckpointError(Exception):
    def __init__(self, path: Path, message: str) -> None:
        super().__init__(message)
        self.path = path


class ModelCheckpointLoader(ABC):
    @abstractmethod
    def lazy_load(self, path: Path, shard_dims: Mapping[str, int], *, gangs: Gangs | None = None, mmap: bool = False,
                  restrict: bool = True, state_dict_converter: StateDictConverter | None = None
                  ) -> Iterator[tuple[str, Tensor]]: ...

    @abstractmethod
    def supports_path(self, path: Path) -> bool: ...


def _target(gangs: Gangs | None) -> tuple[tuple[int, int], tuple[int, int]]:
    if gangs is None:
        return (1, 1), (0, 0)
    return (gangs.tp.size, gangs.sdp.size), (gangs.tp.rank, gangs.sdp.rank)


def _unwrap(sd: dict[str, object]) -> dict[str, object]:
    for k in ("model", "state_dict", "model_state_dict"):
        v = sd.get(k)
        if isinstance(v, dict) and len(sd) <= 8:
            return v
    return sd


class BasicModelCheckpointLoader(ModelCheckpointLoader):
    """A single ``torch.save`` file holding a full (unsharded) state dict."""

    def __init__(self, file_loader: TensorFileLoader | None = None) -> None:
        self._loader = file_loader or TensorFileLoader()

    def supports_path(self, path: Path) -> bool:
        return path.is_file() and path.suffix in (".pt", ".pth", ".bin")

    def lazy_load(self, path, shard_dims, *, gangs=None, mmap=False, restrict=True, state_dict_converter=None):  # type: ignore[override]
        try:
            sd = self._loader.load(path, map_location="cpu", mmap=mmap, restrict=restrict)
        except TensorFileError as ex:
            raise ModelCheckpointError(path, str(ex)) from ex
        sd = _unwrap(sd)
        if state_dict_converter is not None:
            sd = state_dict_converter(sd)
        sizes, ranks = _target(gangs)
        seen: set[int] = set()
        for k, v in sd.items():
            if not isinstance(v, Tensor):
                continue
            yield k, reshard_tensor(k, [[v]], (1, 1), sizes, ranks, shard_dims)


class SafetensorsCheckpointLoader(ModelCheckpointLoader):
    def supports_path(self, path: Path) -> bool:
        if path.is_file():
            return path.suffix == ".safetensors"
        return path.is_dir() and any(path.glob("*.safetensors"))

    def lazy_load(self, path, shard_dims, *, gangs=None, mmap=False, restrict=True, state_dict_converter=None):  # type: ignore[override]
        try:
            sd: dict[str, object] = dict(SafetensorsLoader().load(path, map_location="cpu"))
        except TensorFileError as ex:
            raise ModelCheckpointError(path, str(ex)) from ex
        if state_dict_converter is not None:
            sd = state_dict_converter(sd)
        sizes, ranks = _target(gangs)
        for k, v in sd.items():
            if isinstance(v, Tensor):
                yield k, reshard_tensor(k, [[v]], (1, 1), sizes, ranks, shard_dims)


class NativeModelCheckpointLoader(ModelCheckpointLoader):
    """``<dir>/pp_PP/tp_TT/sdp_SS.pt`` files as written by the checkpoint manager."""

    _RE = re.compile(r"pp_(\d+)/tp_(\d+)/sdp_(\d+)\.pt$")

    def __init__(self, file_loader: TensorFileLoader | None = None) -> None:
        self._loader = file_loader or TensorFileLoader()

    def supports_path(self, path: Path) -> bool:
        return path.is_dir() and (path / "pp_00").is_dir()

    def lazy_load(self, path, shard_dims, *, gangs=None, mmap=False, restrict=True, state_dict_converter=None):  # type: ignore[override]
        files: dict[tuple[int, int], Path] = {}
        for f in sorted(path.glob("pp_*/tp_*/sdp_*.pt")):
            m = self._RE.search(f.as_posix())
            if m is None:
                continue
            if int(m.group(1)) != 0:
                raise ModelCheckpointError(path, "Pipeline-parallel checkpoints are not supported.")
            files[(int(m.group(2)), int(m.group(3)))] = f
        if not files:
            raise ModelCheckpointError(path, f"'{path}' does not contain any model shard file.")
        src_tp = max(t for t, _ in files) + 1
        src_dp = max(d for _, d in files) + 1
        if len(files) != src_tp * src_dp:
            raise ModelCheckpointError(path, f"'{path}' is missing model shard files ({len(files)} of {src_tp * src_dp}).")
        sizes, ranks = _target(gangs)
        # fast path: identical layout -> read only this rank's file
        if (src_tp, src_dp) == sizes:
            sd = self._load(files[ranks], mmap, restrict)
            if state_dict_converter is not None:
                sd = state_dict_converter(sd)
            for k, v in sd.items():
                if isinstance(v, Tensor):
                    yield k, v
            return
        loaded = {key: self._load(f, mmap, restrict) for key, f in files.items()}
        first = loaded[(0, 0)]
        seen: dict[int, str] = {}
        for k in first:
            if not isinstance(first[k], Tensor):
                continue
            splits = [[loaded[(t, d)][k] for d in range(src_dp)] for t in range(src_tp)]
            out = reshard_tensor(k, splits, (src_tp, src_dp), sizes, ranks, shard_dims)
            if state_dict_converter is not None:
                for ck, cv in state_dict_converter({k: out}).items():
                    yield ck, cv  # type: ignore[misc]
            else:
                yield k, out

    def _load(self, f: Path, mmap: bool, restrict: bool) -> dict[str, object]:
        try:
            return self._loader.load(f, map_location="cpu", mmap=mmap, restrict=restrict)
        except TensorFileError as ex:
            raise ModelCheckpointError(f, str(ex)) from ex


class LLaMAModelCheckpointLoader(ModelCheckpointLoader):
    """Meta's reference layout: ``consolidated.NN.pth`` files, one per
    tensor-parallel rank, with the reference key names."""

    def __init__(self, file_loader: TensorFileLoader | None = None) -> None:
        self._loader = file_loader or TensorFileLoader()

    def supports_path(self, path: Path) -> bool:
        return path.is_dir() and any(path.glob("consolidated.*.pth"))

    def lazy_load(self, path, shard_dims, *, gangs=None, mmap=False, restrict=True, state_dict_converter=None):  # type: ignore[override]
        files = sorted(path.glob("consolidated.*.pth"))
        shards = []
        for f in files:
            try:
                sd = self._loader.load(f, map_location="cpu", mmap=mmap, restrict=restrict)
            except TensorFileError as ex:
                raise ModelCheckpointError(f, str(ex)) from ex
            if state_dict_converter is not None:
                sd = state_dict_converter(sd)
            shards.append(sd)
        sizes, ranks = _target(gangs)
        src_tp = len(shards)
        for k, v in shards[0].items():
            if not isinstance(v, Tensor):
                continue
            splits = [[s[k]] for s in shards]
            yield k, reshard_tensor(k, splits, (src_tp, 1), sizes, ranks, shard_dims)


class DelegatingModelCheckpointLoader(ModelCheckpointLoader):
    def __init__(self, loaders: list[ModelCheckpointLoader]) -> None:
        self._loaders = loaders

    def supports_path(self, path: Path) -> bool:
        return any(l.supports_path(path) for l in self._loaders)

    def lazy_load(self, path, shard_dims, **kw):  # type: ignore[override]
        if not path.exists():
            raise ModelCheckpointError(path, f"'{path}' does not exist.")
        for l in self._loaders:
            if l.supports_path(path):
                return l.lazy_load(path, shard_dims, **kw)
        raise ModelCheckpointError(path, f"'{path}' does not point to any known checkpoint format.")


def create_default_checkpoint_loader() -> DelegatingModelCheckpointLoader:
    return DelegatingModelCheckpointLoader([NativeModelCheckpointLoader(), LLaMAModelCheckpointLoader(),
                                            SafetensorsCheckpointLoader(), BasicModelCheckpointLoader()])
