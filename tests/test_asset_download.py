"""Asset download manager against a local HTTP server on 127.0.0.1: staging, length checks, archive extraction with
confinement, cache reuse, ``force`` / ``local_only``, scheme delegation."""
from __future__ import annotations

import io
import tarfile
import threading
import zipfile
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path

import pytest

from fairseq2_b200.assets.download_manager import (AssetDownloadError, AssetDownloadManager, HttpAssetDownloadManager,
                                                   LocalAssetDownloadManager)


def _zip_bytes(members: dict[str, bytes]) -> bytes:
    buf = io.BytesIO()
    with zipfile.ZipFile(buf, "w") as z:
        for n, b in members.items():
            z.writestr(n, b)
    return buf.getvalue()


def _tar_bytes(members: dict[str, bytes]) -> bytes:
    buf = io.BytesIO()
    with tarfile.open(fileobj=buf, mode="w:gz") as t:
        for n, b in members.items():
            info = tarfile.TarInfo(n)
            info.size = len(b)
            t.addfile(info, io.BytesIO(b))
    return buf.getvalue()


ROUTES: dict[str, tuple[bytes, dict[str, str]]] = {
    "/w/model.pt": (b"weights" * 1000, {}),
    "/named": (b"abc", {"Content-Disposition": 'attachment; filename="spm.model"'}),
    "/a/data.zip": (_zip_bytes({"train.jsonl": b"{}\n", "sub/dev.jsonl": b"{}\n"}), {}),
    "/a/data.tar.gz": (_tar_bytes({"x.txt": b"x", "d/y.txt": b"y"}), {}),
    "/a/evil.zip": (_zip_bytes({"../outside.txt": b"no"}), {}),
    "/a/evil.tar": (_tar_bytes({"../../outside.txt": b"no"}), {}),
    "/short": (b"12345", {"Content-Length": "10"}),
}
HITS: dict[str, int] = {}


class _Handler(BaseHTTPRequestHandler):
    def do_GET(self) -> None:  # noqa: N802
        HITS[self.path] = HITS.get(self.path, 0) + 1
        if self.path not in ROUTES:
            self.send_error(404)
            return
        body, headers = ROUTES[self.path]
        self.send_response(200)
        if "Content-Length" not in headers:
            self.send_header("Content-Length", str(len(body)))
        for k, v in headers.items():
            self.send_header(k, v)
        self.end_headers()
        self.wfile.write(body)

    def log_message(self, *a) -> None:  # type: ignore[no-untyped-def]
        pass


@pytest.fixture(scope="module")
def server():  # type: ignore[no-untyped-def]
    srv = ThreadingHTTPServer(("127.0.0.1", 0), _Handler)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield f"http://127.0.0.1:{srv.server_address[1]}"
    srv.shutdown()


def test_single_file_is_cached_and_reused(server: str, tmp_path: Path) -> None:
    dm = AssetDownloadManager(tmp_path)
    uri = server + "/w/model.pt"
    p = dm.download_model(uri, "m")
    assert p.name == "model.pt" and p.read_bytes() == b"weights" * 1000
    n = HITS["/w/model.pt"]
    assert dm.download_model(uri, "m") == p and HITS["/w/model.pt"] == n          # served from the cache
    assert dm.download_model(uri, "m", local_only=True) == p
    assert dm.download_model(uri, "m", force=True) == p and HITS["/w/model.pt"] == n + 1
    assert not list(tmp_path.glob("*.stage-*"))                                    # nothing left behind


def test_content_disposition_names_the_file(server: str, tmp_path: Path) -> None:
    p = AssetDownloadManager(tmp_path).download_tokenizer(server + "/named", "tok")
    assert p.name == "spm.model" and p.read_bytes() == b"abc"


@pytest.mark.parametrize("route,files", [("/a/data.zip", {"train.jsonl", "sub/dev.jsonl"}),
                                         ("/a/data.tar.gz", {"x.txt", "d/y.txt"})])
def test_archives_are_unpacked_into_the_asset_directory(server: str, tmp_path: Path, route: str, files: set[str]) -> None:
    d = AssetDownloadManager(tmp_path).download_dataset(server + route, "ds")
    assert d.is_dir()
    assert {str(p.relative_to(d)) for p in d.rglob("*") if p.is_file()} == files


@pytest.mark.parametrize("route", ["/a/evil.zip", "/a/evil.tar"])
def test_archive_members_cannot_leave_the_cache(server: str, tmp_path: Path, route: str) -> None:
    cache = tmp_path / "cache"
    with pytest.raises(AssetDownloadError, match="outside|cannot be extracted"):
        AssetDownloadManager(cache).download_dataset(server + route, "ds")
    assert not (tmp_path / "outside.txt").exists() and not list(cache.glob("*"))   # nothing cached, nothing staged


def test_errors(server: str, tmp_path: Path) -> None:
    dm = AssetDownloadManager(tmp_path)
    with pytest.raises(AssetDownloadError, match="HTTP 404"):
        dm.download_model(server + "/missing", "m")
    with pytest.raises(AssetDownloadError, match="fewer than"):
        dm.download_model(server + "/short", "m")
    with pytest.raises(AssetDownloadError, match="local_only"):
        dm.download_model(server + "/w/model.pt", "m", local_only=True)
    with pytest.raises(AssetDownloadError, match="not reachable"):
        dm.download_model("http://127.0.0.1:9/none", "m")
    with pytest.raises(AssetDownloadError, match="scheme 'ftp'"):
        dm.download_model("ftp://host/file", "m")
    with pytest.raises(AssetDownloadError, match="not found"):
        dm.download_model(str(tmp_path / "nope.pt"), "m")


def test_local_paths_and_delegation(tmp_path: Path) -> None:
    f = tmp_path / "a b.pt"
    f.write_bytes(b"1")
    dm = AssetDownloadManager(tmp_path)
    assert dm.download_model(str(f), "m") == f
    assert dm.download_model("file://" + str(f).replace(" ", "%20"), "m") == f
    assert dm.supported_schemes == {"", "file", "hg", "http", "https"}
    with pytest.raises(ValueError, match="more than one"):
        AssetDownloadManager(tmp_path, [LocalAssetDownloadManager(), LocalAssetDownloadManager()])
    only_http = AssetDownloadManager(tmp_path, [HttpAssetDownloadManager(tmp_path)])
    with pytest.raises(AssetDownloadError, match="not supported"):
        only_http.download_model(str(f), "m")
