"""File-system abstraction, argparse helpers, pattern sharder."""

from __future__ import annotations

from argparse import ArgumentParser
from pathlib import Path

import pytest
import torch

from fairseq2_b200.file_system import (
    FileMode,
    FileSystemRegistry,
    FSspecFileSystem,
    GlobalFileSystem,
    LocalFileSystem,
    raise_if_not_exists,
)


def _exercise(fs, root: Path) -> None:
    d = root / "a" / "b"
    fs.make_directory(d)
    assert fs.is_dir(d) and not fs.is_file(d)
    with fs.open_text(d / "x.txt", FileMode.WRITE) as fp:
        fp.write("hello")
    with fs.open_text(d / "x.txt", FileMode.APPEND) as fp:
        fp.write(" world")
    assert fs.cat(d / "x.txt") == b"hello world"
    with fs.open(d / "x.txt") as fp:
        assert fp.read() == b"hello world"
    fs.move(d / "x.txt", d / "y.txt")
    assert not fs.exists(d / "x.txt") and fs.is_file(d / "y.txt")
    assert [Path(p).name for p in fs.glob(d, "*.txt")] == ["y.txt"]
    fs.copy_directory(root / "a", root / "c")
    assert fs.cat(root / "c" / "b" / "y.txt") == b"hello world"
    walked = {Path(dp).name: list(names) for dp, names in fs.walk_directory(root / "c", on_error=None)}
    assert walked["b"] == ["y.txt"]
    with fs.tmp_directory(root) as tmp:
        assert fs.is_dir(tmp)
    assert not fs.exists(tmp)
    fs.remove(d / "y.txt")
    fs.remove_directory(root / "c")
    assert not fs.exists(root / "c")
    with pytest.raises(FileNotFoundError):
        raise_if_not_exists(fs, root / "nope")


def test_local_file_system(tmp_path: Path) -> None:
    _exercise(LocalFileSystem(), tmp_path)
    assert LocalFileSystem().is_local


def test_fsspec_and_global_file_system(tmp_path: Path) -> None:
    import fsspec

    _exercise(FSspecFileSystem(fsspec.filesystem("file"), ""), tmp_path / "l")
    FileSystemRegistry.clear()
    FileSystemRegistry.register_protocol("memory")
    try:
        g = GlobalFileSystem()
        _exercise(g, tmp_path / "g")                       # unmatched paths go to the local disk
        _exercise(g, Path("memory://bucket/root"))         # Path collapses '//' -- restored by the adapter
        assert not g.is_local_path(Path("memory://bucket")) and g.is_local_path(tmp_path)
        with pytest.raises(ValueError):
            g.move(tmp_path / "x", Path("memory://bucket/x"))
        src = tmp_path / "up.bin"
        src.write_bytes(b"123")
        g.copy_from_local(src, "memory://bucket/up/up.bin")
        assert g.cat(Path("memory://bucket/up/up.bin")) == b"123"
    finally:
        FileSystemRegistry.clear()


def test_config_action_and_dtype() -> None:
    from fairseq2_b200.utils.argparse import ConfigAction, parse_dtype
    from fairseq2_b200.utils.config import merge_config

    ap = ArgumentParser(exit_on_error=False)
    ap.add_argument("--config", action=ConfigAction, dest="overlays")
    ap.add_argument("--dtype", type=parse_dtype)
    ns = ap.parse_args(["--config", "a.b=1", "set:a.c={x: 2}", "del:d.e", "lr=1e-3", "--dtype", "torch.bfloat16"])
    assert ns.dtype is torch.bfloat16
    (overlay,) = ns.overlays
    assert overlay == {"a": {"_set_": {"b": 1, "c": {"x": 2}}}, "d": {"_del_": ["e"]}, "_set_": {"lr": 1e-3}}
    base = {"a": {"b": 0, "c": {"x": 0, "y": 1}}, "d": {"e": 1, "f": 2}, "lr": 0.1}
    assert merge_config(base, overlay) == {"a": {"b": 1, "c": {"x": 2}}, "d": {"f": 2}, "lr": 1e-3}
    with pytest.raises(Exception):
        ap.parse_args(["--config", "novalue"])
    with pytest.raises(Exception):
        ap.parse_args(["--dtype", "nonsense"])


def test_pattern_sharder() -> None:
    from fairseq2_b200.gang import FakeGang, Gangs
    from fairseq2_b200.nn.embedding import StandardEmbedding, VocabShardedEmbedding
    from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, RowShardedLinear
    from fairseq2_b200.sharder import ShardSpec, ShardSpecError, StandardModelSharder

    class Net(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.embed = StandardEmbedding(16, 8)
            self.up = Linear(8, 32, bias=True)
            self.down = Linear(32, 8, bias=True)
            self.norm = torch.nn.LayerNorm(8)

        def forward(self, x):
            return self.norm(self.down(torch.relu(self.up(self.embed(x)))))

    torch.manual_seed(0)
    net = Net()
    x = torch.randint(0, 16, (2, 5))
    want = net(x)
    root = FakeGang(torch.device("cpu"), rank=0, size=2)
    gangs = Gangs(root=root, dp=FakeGang(torch.device("cpu")), rdp=FakeGang(torch.device("cpu")),
                  sdp=FakeGang(torch.device("cpu")), tp=root, pp=FakeGang(torch.device("cpu")))
    with pytest.warns(DeprecationWarning):
        StandardModelSharder().shard(net, gangs, {r"embed": ShardSpec(0), r"up": ShardSpec(0, region_boundary=True),
                                                  r"down": ShardSpec(1, region_boundary=True)})
    assert isinstance(net.embed, VocabShardedEmbedding) and isinstance(net.up, ColumnShardedLinear)
    assert isinstance(net.down, RowShardedLinear) and net.up.weight.shape == (16, 8) and net.down.weight.shape == (8, 16)
    with pytest.raises(ShardSpecError), pytest.warns(DeprecationWarning):
        StandardModelSharder().shard(net, gangs, {r"norm": ShardSpec(0)})
    del want
