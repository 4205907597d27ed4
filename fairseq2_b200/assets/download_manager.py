"""Resolves asset URIs to local paths (cf. fairseq2
``assets/download_manager.py:40-799``): plain paths and ``file://`` directly,
``hg://org/repo`` through ``huggingface_hub`` (cache-first), ``http(s)://``
into ``~/.cache/fairseq2/assets`` with an atomic rename."""
from __future__ import annotations

import hashlib
import os
import shutil
import urllib.request
from pathlib import Path
from urllib.parse import urlparse


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


class AssetDownloadManager:
    def __init__(self, cache_dir: Path | None = None) -> None:
        self._cache = cache_dir or get_cache_dir()

    def download_model(self, uri: str, name: str, *, force: bool = False, local_only: bool = False) -> Path:
        return self._download(uri, name, "model", force, local_only)

    def download_tokenizer(self, uri: str, name: str, *, force: bool = False, local_only: bool = False) -> Path:
        return self._download(uri, name, "tokenizer", force, local_only)

    def download_dataset(self, uri: str, name: str, *, force: bool = False, local_only: bool = False) -> Path:
        return self._download(uri, name, "dataset", force, local_only)

    def _download(self, uri: str, name: str, kind: str, force: bool, local_only: bool) -> Path:
        p = urlparse(uri)
        if p.scheme in ("", "file"):
            path = Path(p.netloc + p.path if p.scheme == "file" else uri).expanduser()
            if not path.exists():
                raise AssetDownloadError(uri, f"The {kind} of '{name}' is not found at '{path}'.")
            return path
        if p.scheme == "hg":
            repo = (p.netloc + p.path).strip("/")
            try:
                from huggingface_hub import snapshot_download
            except ImportError as ex:
                raise AssetDownloadError(uri, "huggingface_hub is required for hg:// URIs.") from ex
            try:
                return Path(snapshot_download(repo, local_files_only=local_only))
            except Exception as ex:  # noqa: BLE001
                raise AssetDownloadError(uri, f"The {kind} of '{name}' cannot be downloaded from the Hugging Face Hub: {ex}") from ex
        if p.scheme in ("http", "https"):
            h = hashlib.sha1(uri.encode()).hexdigest()[:24]
            target = self._cache / h / Path(p.path).name
            if target.exists() and not force:
                return target
            if local_only:
                raise AssetDownloadError(uri, f"The {kind} of '{name}' is not in the local cache.")
            target.parent.mkdir(parents=True, exist_ok=True)
            tmp = target.with_suffix(target.suffix + ".part")
            try:
                with urllib.request.urlopen(uri) as r, tmp.open("wb") as fp:
                    shutil.copyfileobj(r, fp)
                tmp.replace(target)
            except OSError as ex:
                raise AssetDownloadError(uri, f"The {kind} of '{name}' cannot be downloaded: {ex}") from ex
            return target
        raise AssetDownloadError(uri, f"The URI scheme '{p.scheme}' of the {kind} of '{name}' is not supported.")
