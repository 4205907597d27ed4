"""File-system abstraction: one interface over the local disk and fsspec back ends.

``FileSystem`` is the interface every component that touches storage (tensor
IO, checkpoint manager, asset store, recipes) is written against.
``LocalFileSystem`` implements it with ``os``/``shutil``; ``FSspecFileSystem``
adapts any fsspec file system (S3 and the like) under a URI prefix;
``GlobalFileSystem`` looks at each path and forwards to whichever registered
file system claims it, so callers can pass ``s3://bucket/x`` and ``/data/x``
to the same object.

Mirrors the surface of fairseq2 ``file_system.py:33-695`` (``FileMode``,
``FileSystem``, ``FSspecFileSystem``, ``FileSystemRegistry``,
``GlobalFileSystem``, ``NativeLocalFileSystem``, ``raise_if_not_exists``,
NFS lookup-cache flush before reads).
"""

from __future__ import annotations

import os
import shutil
import tempfile
from abc import ABC, abstractmethod
from collections.abc import Callable, Iterator, Sequence
from contextlib import contextmanager
from enum import Enum
from errno import ENOENT
from pathlib import Path
from typing import Any, BinaryIO, ContextManager, TextIO, cast


class FileMode(Enum):
    READ = 0
    WRITE = 1
    APPEND = 2


_BINARY_MODES = {FileMode.READ: "rb", FileMode.WRITE: "wb", FileMode.APPEND: "ab"}
_TEXT_MODES = {FileMode.READ: "r", FileMode.WRITE: "w", FileMode.APPEND: "a"}


class FileSystem(ABC):
    @abstractmethod
    def is_file(self, path: Path) -> bool: ...

    @abstractmethod
    def is_dir(self, path: Path) -> bool: ...

    @abstractmethod
    def open(self, path: Path, mode: FileMode = FileMode.READ) -> BinaryIO: ...

    @abstractmethod
    def open_text(self, path: Path, mode: FileMode = FileMode.READ) -> TextIO: ...

    def cat(self, path: Path) -> bytes:
        with self.open(path) as fp:
            return fp.read()

    @abstractmethod
    def exists(self, path: Path) -> bool: ...

    @abstractmethod
    def move(self, old_path: Path, new_path: Path) -> None: ...

    @abstractmethod
    def remove(self, path: Path) -> None: ...

    @abstractmethod
    def make_directory(self, path: Path) -> None: ...

    @abstractmethod
    def copy_directory(self, source_path: Path, target_path: Path) -> None: ...

    def copy_from_local(self, local_path: Path, remote_path: Path | str) -> None:
        """Upload a local file or directory; on a local file system this is a plain copy."""
        target = Path(remote_path)
        if Path(local_path).is_dir():
            self.copy_directory(Path(local_path), target)
        else:
            self.make_directory(target.parent)
            with open(local_path, "rb") as src, self.open(target, FileMode.WRITE) as dst:
                shutil.copyfileobj(src, dst)

    @abstractmethod
    def remove_directory(self, path: Path) -> None: ...

    @abstractmethod
    def glob(self, path: Path, pattern: str) -> Iterator[Path]: ...

    @abstractmethod
    def walk_directory(self, path: Path, *, on_error: Callable[[OSError], None] | None) -> Iterator[tuple[str, Sequence[str]]]:
        """Yield ``(dir_path, file_names)`` pairs top-down."""

    @abstractmethod
    def tmp_directory(self, base_dir: Path) -> ContextManager[Path]: ...

    @abstractmethod
    def resolve(self, path: Path) -> Path: ...

    @property
    @abstractmethod
    def is_local(self) -> bool: ...

    def is_local_path(self, path: Path) -> bool:  # noqa: ARG002
        return self.is_local


def flush_nfs_lookup_cache(path: Path) -> None:
    """Drop cached NFS LOOKUP results for ``path`` by listing its nearest existing ancestor directory.

    A rank that polls for a file another node just wrote can otherwise keep seeing a stale negative entry
    (fairseq2 ``file_system.py:675-695``).
    """
    path = Path(path)
    while path != path.parent:
        try:
            it = os.scandir(path)
        except (FileNotFoundError, NotADirectoryError):
            path = path.parent
            continue
        except OSError:
            return
        with it:
            next(it, None)
        return


class NativeLocalFileSystem(FileSystem):
    """The local disk through ``os`` / ``shutil``."""

    def is_file(self, path: Path) -> bool:
        flush_nfs_lookup_cache(path)
        return Path(path).is_file()

    def is_dir(self, path: Path) -> bool:
        flush_nfs_lookup_cache(path)
        return Path(path).is_dir()

    def open(self, path: Path, mode: FileMode = FileMode.READ) -> BinaryIO:
        if mode == FileMode.READ:
            flush_nfs_lookup_cache(path)
        return cast(BinaryIO, Path(path).open(_BINARY_MODES[mode]))

    def open_text(self, path: Path, mode: FileMode = FileMode.READ) -> TextIO:
        if mode == FileMode.READ:
            flush_nfs_lookup_cache(path)
        return cast(TextIO, Path(path).open(_TEXT_MODES[mode], encoding="utf-8"))

    def cat(self, path: Path) -> bytes:
        flush_nfs_lookup_cache(path)
        return Path(path).read_bytes()

    def exists(self, path: Path) -> bool:
        flush_nfs_lookup_cache(path)
        return Path(path).exists()

    def move(self, old_path: Path, new_path: Path) -> None:
        Path(old_path).replace(new_path)

    def remove(self, path: Path) -> None:
        Path(path).unlink()

    def make_directory(self, path: Path) -> None:
        Path(path).mkdir(parents=True, exist_ok=True)

    def copy_directory(self, source_path: Path, target_path: Path) -> None:
        shutil.copytree(source_path, target_path, dirs_exist_ok=True)

    def remove_directory(self, path: Path) -> None:
        shutil.rmtree(path)

    def glob(self, path: Path, pattern: str) -> Iterator[Path]:
        return Path(path).glob(pattern)

    def walk_directory(self, path: Path, *, on_error: Callable[[OSError], None] | None) -> Iterator[tuple[str, Sequence[str]]]:
        for dir_path, _, file_names in os.walk(path, onerror=on_error):
            yield dir_path, file_names

    @contextmanager
    def tmp_directory(self, base_dir: Path) -> Iterator[Path]:
        with tempfile.TemporaryDirectory(dir=base_dir) as name:
            yield Path(name)

    def resolve(self, path: Path) -> Path:
        return Path(path).expanduser().resolve()

    @property
    def is_local(self) -> bool:
        return True


LocalFileSystem = NativeLocalFileSystem


class FSspecFileSystem(FileSystem):
    """Adapter over an ``fsspec.AbstractFileSystem``. ``prefix`` is the URI scheme with ``://`` (empty for local).

    ``pathlib.Path`` collapses ``s3://bucket`` to ``s3:/bucket``; ``get_long_uri`` restores the full form before a
    path is handed to fsspec and ``get_short_uri`` strips the scheme from what fsspec returns.
    """

    def __init__(self, fs: Any, prefix: str) -> None:
        self._fs = fs
        self._prefix = prefix
        self._scheme = prefix.split("://")[0] if prefix else ""

    def _bare(self, path: Path | str) -> str:
        s = str(path)
        if self._scheme:
            for head in (self._scheme + "://", self._scheme + ":/"):
                if s.startswith(head):
                    return s[len(head):].lstrip("/") if head.endswith("://") else s[len(head):].lstrip("/")
        return s

    def get_short_uri(self, path: Path | str | Sequence[Path | str]) -> str | list[str]:
        if isinstance(path, (str, Path)):
            return self._bare(path)
        return [self._bare(p) for p in path]

    def get_long_uri(self, path: Path | str | Sequence[Path | str]) -> str | list[str]:
        if isinstance(path, (str, Path)):
            return self._prefix + self._bare(path)
        return [self._prefix + self._bare(p) for p in path]

    def _u(self, path: Path | str) -> str:
        return cast(str, self.get_long_uri(path))

    def _p(self, s: str) -> Path:
        return Path(self._prefix + self._bare(s)) if self._prefix else Path(s)

    def is_file(self, path: Path) -> bool:
        return bool(self._fs.isfile(self._u(path)))

    def is_dir(self, path: Path) -> bool:
        return bool(self._fs.isdir(self._u(path)))

    def exists(self, path: Path) -> bool:
        return bool(self._fs.exists(self._u(path)))

    def open(self, path: Path, mode: FileMode = FileMode.READ) -> BinaryIO:
        return cast(BinaryIO, self._fs.open(self._u(path), _BINARY_MODES[mode]))

    def open_text(self, path: Path, mode: FileMode = FileMode.READ) -> TextIO:
        return cast(TextIO, self._fs.open(self._u(path), _TEXT_MODES[mode], encoding="utf-8"))

    def cat(self, path: Path) -> bytes:
        return cast(bytes, self._fs.cat_file(self._u(path)))

    def move(self, old_path: Path, new_path: Path) -> None:
        self._fs.mv(self._u(old_path), self._u(new_path), recursive=True)

    def remove(self, path: Path) -> None:
        self._fs.rm_file(self._u(path))

    def make_directory(self, path: Path) -> None:
        self._fs.makedirs(self._u(path), exist_ok=True)

    def copy_directory(self, source_path: Path, target_path: Path) -> None:
        self._fs.copy(self._u(source_path).rstrip("/") + "/", self._u(target_path).rstrip("/") + "/", recursive=True)

    def copy_from_local(self, local_path: Path, remote_path: Path | str) -> None:
        local = Path(local_path)
        if not local.exists():
            raise FileNotFoundError(ENOENT, os.strerror(ENOENT), str(local))
        self._fs.put(str(local), self._u(remote_path), recursive=local.is_dir())

    def remove_directory(self, path: Path) -> None:
        self._fs.rm(self._u(path), recursive=True)

    def glob(self, path: Path, pattern: str) -> Iterator[Path]:
        for s in self._fs.glob(self._u(path).rstrip("/") + "/" + pattern):
            yield self._p(s)

    def walk_directory(self, path: Path, *, on_error: Callable[[OSError], None] | None) -> Iterator[tuple[str, Sequence[str]]]:
        kw = {"on_error": on_error} if on_error is not None else {}
        for dir_path, _, file_names in self._fs.walk(self._u(path), **kw):
            yield str(self._p(dir_path)), file_names

    @contextmanager
    def tmp_directory(self, base_dir: Path) -> Iterator[Path]:
        name = Path(self._u(base_dir).rstrip("/") + "/tmp_" + os.urandom(8).hex())
        self.make_directory(name)
        try:
            yield name
        finally:
            try:
                self.remove_directory(name)
            except (OSError, FileNotFoundError):
                pass

    def resolve(self, path: Path) -> Path:
        if self.is_local:
            return Path(path).expanduser().resolve()
        return self._p(str(path))

    @property
    def is_local(self) -> bool:
        protocol = getattr(self._fs, "protocol", ())
        protocols = (protocol,) if isinstance(protocol, str) else tuple(protocol)
        return not self._prefix and ("file" in protocols or "local" in protocols)


PathOrPaths = Any


class FileSystemRegistry:
    """Ordered ``(matches(path), factory)`` rules; the first match wins, unmatched paths are local."""

    _resolvers: list[tuple[Callable[[str], bool], Callable[[], FileSystem]]] = []
    _fs_cache: dict[Any, FileSystem] = {}
    _local_fs: FileSystem = NativeLocalFileSystem()

    @classmethod
    def register(cls, pattern_check: Callable[[str], bool], fs_factory: Callable[[], FileSystem]) -> None:
        cls._resolvers.append((pattern_check, fs_factory))

    @classmethod
    def register_protocol(cls, protocol: str, **storage_options: Any) -> None:
        """Route ``protocol://…`` (also the ``protocol:/…`` form ``Path`` produces) to the fsspec back end of that name."""

        def check(path: str) -> bool:
            return path.startswith(protocol + "://") or path.startswith(protocol + ":/")

        def factory() -> FileSystem:
            import fsspec

            return FSspecFileSystem(fsspec.filesystem(protocol, **storage_options), protocol + "://")

        cls.register(check, factory)

    @classmethod
    def clear(cls) -> None:
        cls._resolvers = []
        cls._fs_cache = {}

    @classmethod
    def resolve_filesystem(cls, path: PathOrPaths) -> FileSystem:
        if isinstance(path, Sequence) and not isinstance(path, (str, Path)):
            if not path:
                return cls._local_fs
            fs = cls.resolve_filesystem(path[0])
            for p in path[1:]:
                if cls.resolve_filesystem(p) is not fs:
                    raise ValueError("The paths of the sequence resolve to different file systems.")
            return fs
        s = str(path)
        for check, factory in cls._resolvers:
            if check(s):
                fs = cls._fs_cache.get(check)
                if fs is None:
                    fs = cls._fs_cache[check] = factory()
                return fs
        return cls._local_fs


class GlobalFileSystem(FileSystem):
    """Forwards every call to the file system that ``FileSystemRegistry`` resolves for the path."""

    @staticmethod
    def _of(path: PathOrPaths) -> FileSystem:
        return FileSystemRegistry.resolve_filesystem(path)

    def is_file(self, path: Path) -> bool:
        return self._of(path).is_file(path)

    def is_dir(self, path: Path) -> bool:
        return self._of(path).is_dir(path)

    def open(self, path: Path, mode: FileMode = FileMode.READ) -> BinaryIO:
        return self._of(path).open(path, mode)

    def open_text(self, path: Path, mode: FileMode = FileMode.READ) -> TextIO:
        return self._of(path).open_text(path, mode)

    def cat(self, path: Path) -> bytes:
        return self._of(path).cat(path)

    def exists(self, path: Path) -> bool:
        return self._of(path).exists(path)

    def move(self, old_path: Path, new_path: Path) -> None:
        self._of([old_path, new_path]).move(old_path, new_path)

    def remove(self, path: Path) -> None:
        self._of(path).remove(path)

    def make_directory(self, path: Path) -> None:
        self._of(path).make_directory(path)

    def copy_directory(self, source_path: Path, target_path: Path) -> None:
        self._of([source_path, target_path]).copy_directory(source_path, target_path)

    def copy_from_local(self, local_path: Path, remote_path: Path | str) -> None:
        self._of(remote_path).copy_from_local(local_path, remote_path)

    def remove_directory(self, path: Path) -> None:
        self._of(path).remove_directory(path)

    def glob(self, path: Path, pattern: str) -> Iterator[Path]:
        return self._of(path).glob(path, pattern)

    def walk_directory(self, path: Path, *, on_error: Callable[[OSError], None] | None) -> Iterator[tuple[str, Sequence[str]]]:
        return self._of(path).walk_directory(path, on_error=on_error)

    def tmp_directory(self, base_dir: Path) -> ContextManager[Path]:
        return self._of(base_dir).tmp_directory(base_dir)

    def resolve(self, path: Path) -> Path:
        return self._of(path).resolve(path)

    @property
    def is_local(self) -> bool:
        return False

    def is_local_path(self, path: Path) -> bool:
        return self._of(path).is_local


def raise_if_not_exists(file_system: FileSystem, path: Path) -> None:
    if not file_system.exists(path):
        raise FileNotFoundError(ENOENT, os.strerror(ENOENT), str(path))
