"""Resolves asset URIs to local paths (cf. fairseq2 ``assets/download_manager.py:40-799``).

``AssetDownloadManager()`` is the entry point; it hands a URI to the manager that knows its scheme:

* :class:`LocalAssetDownloadManager` -- plain paths and ``file://``;
* :class:`HuggingFaceHub` -- ``hg://org/repo`` through ``huggingface_hub`` (cache-first, per-kind file patterns);
* :class:`HttpAssetDownloadManager` -- ``http(s)://`` into ``<cache>/<sha1(uri)[:24]>/``.

An HTTP download is staged: the body is streamed into ``<hash>.stage-<pid>/`` (length checked against
``Content-Length``, file name from ``Content-Disposition`` or the final URL), ``.zip`` files and tar archives are
unpacked there with every member confined to the stage directory, and only then the directory is renamed to
``<hash>/``. A crash therefore never leaves a half-written asset in the cache, and concurrent downloads of one URI
(several ranks of a job) end with one winner and identical content. The returned path is the single file of the
asset directory if there is exactly one, else the directory. ``force`` drops the cached copy first; ``local_only``
never touches the network.
"""
from __future__ import annotations

import hashlib
import os
import re
import shutil
import tarfile
import urllib.error
import urllib.request
import zipfile
from abc import ABC, abstractmethod
from collections.abc import Sequence
from pathlib import Path
from urllib.parse import unquote, urlparse

from fairseq2_b200.logging import log


class AssetDownloadError(Exception):
    def __init__(self, uri: str, message: str) -> None:
        super().__init__(message)
        self.uri = uri


def get_cache_dir() -> Path:
    d = os.environ.get("FAIRSEQ2_CACHE_DIR")
    if d:
        return Path(d).expanduser()
    xdg = os.environ.get("XDG_CACHE_HOME")
    return (Path(xdg) if xdg else Path("~/.cache").expanduser()) / "fairseq2" / "assets"


class _SchemeManager(ABC):
    """One URI scheme family. ``kind`` is "model", "tokenizer" or "dataset"."""

    @property
    @abstractmethod
    def supported_schemes(self) -> set[str]: ...

    @abstractmethod
    def fetch(self, uri: str, name: str, kind: str, *, force: bool, local_only: bool) -> Path: ...


class LocalAssetDownloadManager(_SchemeManager):
    @property
    def supported_schemes(self) -> set[str]:
        return {"", "file"}

    def fetch(self, uri: str, name: str, kind: str, *, force: bool, local_only: bool) -> Path:
        p = urlparse(uri)
        path = Path(unquote(p.netloc + p.path) if p.scheme == "file" else uri).expanduser()
        if not path.exists():
            raise AssetDownloadError(uri, f"The {kind} of '{name}' is not found at '{path}'.")
        return path


class HuggingFaceHub(_SchemeManager):
    """``hg://org/repo[@revision]``. Models fetch weight and config files only, tokenizers their vocabulary files,
    datasets use the dataset repository type."""

    _PATTERNS = {
        "model": ["*.safetensors", "*.safetensors.index.json", "*.bin", "*.bin.index.json", "*.pt", "*.pth", "*.json"],
        "tokenizer": ["tokenizer*", "*.model", "*.tiktoken", "vocab*", "merges.txt", "special_tokens_map.json",
                      "added_tokens.json", "*.json"],
        "dataset": None,
    }

    @property
    def supported_schemes(self) -> set[str]:
        return {"hg"}

    def fetch(self, uri: str, name: str, kind: str, *, force: bool, local_only: bool) -> Path:
        p = urlparse(uri)
        repo = (p.netloc + p.path).strip("/")
        revision = None
        if "@" in repo:
            repo, revision = repo.rsplit("@", 1)
        if repo.count("/") > 1 or not repo:
            raise AssetDownloadError(uri, f"'{uri}' is not of the form hg://[org/]repo[@revision].")
        try:
            from huggingface_hub import snapshot_download
        except ImportError as ex:
            raise AssetDownloadError(uri, "huggingface_hub is required for hg:// URIs.") from ex
        try:
            return Path(snapshot_download(repo, revision=revision, local_files_only=local_only, force_download=force,
                                          allow_patterns=self._PATTERNS[kind],
                                          repo_type="dataset" if kind == "dataset" else None))
        except Exception as ex:  # noqa: BLE001 - the hub raises a family of errors of its own
            raise AssetDownloadError(
                uri, f"The {kind} of '{name}' cannot be downloaded from the Hugging Face Hub: {ex}") from ex


class HttpAssetDownloadManager(_SchemeManager):
    _CHUNK = 1 << 16
    # most hosting providers answer 403 to an unknown client string
    _AGENT = "Mozilla/5.0 (X11; Linux x86_64; rv:109.0) Gecko/20100101 Firefox/119.0"

    def __init__(self, cache_dir: Path | None = None, *, progress: bool = True) -> None:
        self._cache = cache_dir or get_cache_dir()
        self._progress = progress

    @property
    def supported_schemes(self) -> set[str]:
        return {"http", "https"}

    def asset_dir(self, uri: str) -> Path:
        return self._cache / hashlib.sha1(uri.encode()).hexdigest()[:24]

    def fetch(self, uri: str, name: str, kind: str, *, force: bool, local_only: bool) -> Path:
        final = self.asset_dir(uri)
        try:
            if force and not local_only:
                shutil.rmtree(final, ignore_errors=True)
            if not final.exists():
                if local_only:
                    raise AssetDownloadError(uri, f"The {kind} of '{name}' is not cached, but `local_only` is set.")
                self._download_into_cache(uri, name, kind, final)
            return self._asset_path(uri, final)
        except OSError as ex:
            raise AssetDownloadError(uri, f"The {kind} of '{name}' cannot be downloaded: {ex}") from ex

    def _download_into_cache(self, uri: str, name: str, kind: str, final: Path) -> None:
        stage = final.with_name(f"{final.name}.stage-{os.getpid()}")
        shutil.rmtree(stage, ignore_errors=True)
        stage.mkdir(parents=True)
        try:
            body = self._stream(uri, name, kind, stage)
            self._unpack(uri, body, stage)
            try:
                stage.rename(final)
            except OSError:
                if not final.exists():          # not a lost race against another process: a real failure
                    raise
        finally:
            shutil.rmtree(stage, ignore_errors=True)

    def _stream(self, uri: str, name: str, kind: str, stage: Path) -> Path:
        request = urllib.request.Request(uri, headers={"User-Agent": self._AGENT})
        try:
            response = urllib.request.urlopen(request)
        except urllib.error.HTTPError as ex:
            raise AssetDownloadError(uri, f"The server answered HTTP {ex.code} for the {kind} of '{name}'.") from ex
        except urllib.error.URLError as ex:
            raise AssetDownloadError(uri, f"The address of the {kind} of '{name}' is not reachable: {ex.reason}") from ex
        with response:
            expected = None
            length = response.headers.get("Content-Length")
            if length is not None and length.isdigit():
                expected = int(length)
            filename = None
            disposition = response.headers.get("Content-Disposition")
            if disposition:
                m = re.search(r"filename\*?=(?:UTF-8'')?\"?([^\";\n]+)\"?", disposition)
                if m:
                    filename = Path(unquote(m.group(1))).name
            if not filename:
                filename = Path(unquote(urlparse(response.geturl()).path)).name or "asset"
            target = stage / filename
            task = self._progress_task(f"download {name}", expected)
            received = 0
            try:
                with target.open("wb") as fp:
                    while True:
                        chunk = response.read(self._CHUNK)
                        if not chunk:
                            break
                        received += len(chunk)
                        if expected is not None and received > expected:
                            raise AssetDownloadError(
                                uri, f"The server sent more than the announced {expected:,} bytes.")
                        fp.write(chunk)
                        if task is not None:
                            task.step(len(chunk))
            finally:
                if task is not None:
                    task.close()
            if expected is not None and received < expected:
                raise AssetDownloadError(
                    uri, f"The server sent {received:,} bytes, fewer than the announced {expected:,} bytes.")
        return target

    def _progress_task(self, label: str, total: int | None):  # type: ignore[no-untyped-def]
        if not self._progress or os.environ.get("FAIRSEQ2_NO_PROGRESS"):
            return None
        try:
            from fairseq2_b200.utils.progress import TqdmProgressReporter

            return TqdmProgressReporter().create_task(label, total)
        except Exception:  # noqa: BLE001 - progress output is best effort
            return None

    @staticmethod
    def _unpack(uri: str, body: Path, stage: Path) -> None:
        """Archives are unpacked next to themselves and removed. Only ``.zip`` suffixes count as zip archives:
        several tensor file formats are zip containers and must stay files."""
        root = stage.resolve()

        def confined(member: str) -> None:
            dest = (stage / member).resolve()
            if dest != root and root not in dest.parents:
                raise AssetDownloadError(uri, f"The archive member '{member}' would be written outside the cache.")

        try:
            if body.suffix == ".zip":
                with zipfile.ZipFile(body) as zf:
                    for member in zf.namelist():
                        confined(member)
                    zf.extractall(stage)
                body.unlink()
            elif tarfile.is_tarfile(body):
                with tarfile.open(body) as tf:
                    for m in tf.getmembers():
                        confined(m.name)
                        if m.issym() or m.islnk():
                            confined(os.path.join(os.path.dirname(m.name), m.linkname))
                    tf.extractall(stage, filter="data")
                body.unlink()
        except (zipfile.BadZipFile, tarfile.TarError, EOFError, KeyError) as ex:
            raise AssetDownloadError(uri, f"'{body.name}' cannot be extracted: {ex}") from ex

    @staticmethod
    def _asset_path(uri: str, final: Path) -> Path:
        entries = sorted(final.iterdir())
        if not entries:
            raise AssetDownloadError(uri, f"The asset directory '{final}' is empty.")
        if len(entries) == 1 and entries[0].is_file():
            return entries[0]
        return final


StandardAssetDownloadManager = HttpAssetDownloadManager


class AssetDownloadManager:
    """Delegates to the manager of the URI's scheme (the default set covers local paths, ``hg://`` and ``http(s)://``)."""

    def __init__(self, cache_dir: Path | None = None, managers: Sequence[_SchemeManager] | None = None) -> None:
        if managers is None:
            managers = [LocalAssetDownloadManager(), HuggingFaceHub(), HttpAssetDownloadManager(cache_dir)]
        self._by_scheme: dict[str, _SchemeManager] = {}
        for m in managers:
            for scheme in m.supported_schemes:
                if scheme in self._by_scheme:
                    raise ValueError(f"The URI scheme '{scheme}' is claimed by more than one download manager.")
                self._by_scheme[scheme] = m

    @property
    def supported_schemes(self) -> set[str]:
        return set(self._by_scheme)

    def download_model(self, uri: str, name: str, *, force: bool = False, local_only: bool = False) -> Path:
        return self._download(uri, name, "model", force, local_only)

    def download_tokenizer(self, uri: str, name: str, *, force: bool = False, local_only: bool = False) -> Path:
        return self._download(uri, name, "tokenizer", force, local_only)

    def download_dataset(self, uri: str, name: str, *, force: bool = False, local_only: bool = False) -> Path:
        return self._download(uri, name, "dataset", force, local_only)

    def _download(self, uri: str, name: str, kind: str, force: bool, local_only: bool) -> Path:
        scheme = urlparse(uri).scheme
        if len(scheme) == 1:                      # a Windows drive letter, not a scheme
            scheme = ""
        manager = self._by_scheme.get(scheme)
        if manager is None:
            raise AssetDownloadError(uri, f"The URI scheme '{scheme}' of the {kind} of '{name}' is not supported "
                                          f"(known: {', '.join(sorted(s or 'path' for s in self._by_scheme))}).")
        path = manager.fetch(uri, name, kind, force=force, local_only=local_only)
        log.debug("The {} of '{}' resolved to {}.", kind, name, path)
        return path


DelegatingAssetDownloadManager = AssetDownloadManager


def get_asset_download_manager() -> AssetDownloadManager:
    return AssetDownloadManager()
