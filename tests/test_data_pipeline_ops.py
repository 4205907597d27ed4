"""One contract check per data-pipeline operator: the full output, a ``state_dict`` round trip at every split point
(into the same pipeline and into a freshly built one), and ``reset()`` (cf. the per-operator files of fairseq2's
``tests/unit/data/data_pipeline/``)."""
from __future__ import annotations

import pickle
from pathlib import Path
from typing import Any, Callable

import pytest
import torch

from fairseq2_b200.data import DataPipeline, read_sequence, read_zipped_records
from fairseq2_b200.data.data_pipeline import DataPipelineError
from fairseq2_b200.data.text import read_text


def _norm(x: Any) -> Any:
    if isinstance(x, torch.Tensor):
        return ("tensor", tuple(x.shape), x.flatten().tolist())
    if isinstance(x, (list, tuple)):
        return [_norm(e) for e in x]
    if isinstance(x, dict):
        return {k: _norm(v) for k, v in x.items()}
    if isinstance(x, memoryview):
        return bytes(x)
    return x


def _drain(p: DataPipeline) -> list[Any]:
    return [_norm(x) for x in p]


def _seq(n: int, start: int = 0) -> list[int]:
    return list(range(start, start + n))


def _text_file(tmp: Path) -> Path:
    f = tmp / "lines.txt"
    f.write_text("".join(f"line {i}\n" for i in range(9)))
    return f


def _zip_file(tmp: Path) -> Path:
    import zipfile

    f = tmp / "records.zip"
    with zipfile.ZipFile(f, "w", zipfile.ZIP_DEFLATED) as z:
        for i in range(5):
            z.writestr(f"r{i}.bin", bytes([i]) * (i + 1))
    return f


Builders = dict[str, Callable[[Path], DataPipeline]]

OPERATORS: Builders = {
    "read_sequence": lambda t: read_sequence(_seq(6)).and_return(),
    "bucket": lambda t: read_sequence(_seq(11)).bucket(4).and_return(),
    "bucket_drop_remainder": lambda t: read_sequence(_seq(11)).bucket(4, drop_remainder=True).and_return(),
    "bucket_by_length": lambda t: read_sequence([torch.zeros(n) for n in (1, 3, 2, 4, 1, 2, 3, 4, 1)])
    .bucket_by_length([(3, 2), (2, 4)]).and_return(),
    "dynamic_bucket": lambda t: read_sequence(_seq(12, 1)).dynamic_bucket(10, lambda x: float(x)).and_return(),
    "filter": lambda t: read_sequence(_seq(15)).filter(lambda x: x % 3 != 0).and_return(),
    "map": lambda t: read_sequence(_seq(9)).map(lambda x: x * x).and_return(),
    "map_parallel": lambda t: read_sequence(_seq(25)).map(lambda x: x + 1, num_parallel_calls=4).and_return(),
    "map_selector": lambda t: read_sequence([{"a": i, "b": [i, i]} for i in range(6)])
    .map(lambda x: x * 10, selector="a,b[1]").and_return(),
    "pack": lambda t: read_sequence([torch.arange(n) for n in (3, 5, 2, 7, 1, 4, 6)])
    .pack(num_elements=8, max_seq_len=6, pad_value=0).and_return(),
    "prefetch": lambda t: read_sequence(_seq(20)).prefetch(3).and_return(),
    "repeat": lambda t: read_sequence(_seq(3)).repeat(3).and_return(),
    "shard": lambda t: read_sequence(_seq(13)).shard(1, 3).and_return(),
    "shard_uneven": lambda t: read_sequence(_seq(13)).shard(0, 3, allow_uneven=True).and_return(),
    "shuffle": lambda t: read_sequence(_seq(30)).shuffle(8, seed=5).and_return(),
    "shuffle_full": lambda t: read_sequence(_seq(12)).shuffle(0, seed=5).and_return(),
    "skip": lambda t: read_sequence(_seq(8)).skip(3).and_return(),
    "take": lambda t: read_sequence(_seq(8)).take(5).and_return(),
    "yield_from": lambda t: read_sequence(_seq(4, 1)).yield_from(lambda n: read_sequence(_seq(n, 10 * n)).and_return())
    .and_return(),
    "concat": lambda t: DataPipeline.concat([read_sequence(_seq(3)).and_return(),
                                             read_sequence(_seq(4, 10)).and_return()]).and_return(),
    "constant": lambda t: DataPipeline.constant(7).take(4).and_return(),
    "count": lambda t: DataPipeline.count(3, step=2).take(6).and_return(),
    "round_robin": lambda t: DataPipeline.round_robin([read_sequence(_seq(5)).and_return(),
                                                       read_sequence(_seq(2, 100)).and_return()]).and_return(),
    "round_robin_shortest": lambda t: DataPipeline.round_robin(
        [read_sequence(_seq(5)).and_return(), read_sequence(_seq(2, 100)).and_return()],
        stop_at_shortest=True).and_return(),
    "sample": lambda t: DataPipeline.sample([read_sequence(_seq(6)).and_return(),
                                             read_sequence(_seq(9, 100)).and_return()], weights=[0.3, 0.7],
                                            seed=11).and_return(),
    "zip": lambda t: DataPipeline.zip([read_sequence(_seq(5)).and_return(), read_sequence(_seq(5, 50)).and_return()],
                                      names=["x", "y"]).and_return(),
    "zip_flatten": lambda t: DataPipeline.zip(
        [read_sequence([{"a": i} for i in range(4)]).and_return(),
         read_sequence([{"b": -i} for i in range(4)]).and_return()], flatten=True).and_return(),
    "read_text": lambda t: read_text(_text_file(t), rtrim=True).and_return(),
    "read_text_mmap": lambda t: read_text(_text_file(t), rtrim=True, memory_map=True).and_return(),
    "read_zipped_records": lambda t: read_zipped_records(_zip_file(t)).map(lambda b: bytes(b)).and_return(),
    "composite": lambda t: read_sequence(_seq(40)).shuffle(10, seed=1).filter(lambda x: x % 5 != 0)
    .map(lambda x: torch.full((x % 4 + 1,), x), num_parallel_calls=2).bucket(3).prefetch(2).and_return(),
}

EXPECTED: dict[str, Any] = {
    "read_sequence": _seq(6),
    "bucket": [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10]],
    "bucket_drop_remainder": [[0, 1, 2, 3], [4, 5, 6, 7]],
    "filter": [x for x in _seq(15) if x % 3],
    "map": [x * x for x in _seq(9)],
    "map_parallel": _seq(25, 1),
    "map_selector": [{"a": i * 10, "b": [i, i * 10]} for i in range(6)],
    "prefetch": _seq(20),
    "repeat": _seq(3) * 3,
    "shard": [1, 4, 7, 10],
    "shard_uneven": [0, 3, 6, 9, 12],
    "skip": _seq(5, 3),
    "take": _seq(5),
    "yield_from": [10, 20, 21, 30, 31, 32, 40, 41, 42, 43],
    "concat": [0, 1, 2, 10, 11, 12, 13],
    "constant": [7] * 4,
    "count": [3, 5, 7, 9, 11, 13],
    "round_robin": [0, 100, 1, 101, 2, 100, 3, 101, 4, 100],
    "round_robin_shortest": [0, 100, 1, 101],
    "zip": [{"x": i, "y": 50 + i} for i in range(5)],
    "zip_flatten": [{"a": i, "b": -i} for i in range(4)],
    "read_text": [f"line {i}" for i in range(9)],
    "read_text_mmap": [f"line {i}" for i in range(9)],
    "read_zipped_records": [bytes([i]) * (i + 1) for i in range(5)],
}


@pytest.mark.parametrize("name", sorted(OPERATORS))
def test_operator_output(name: str, tmp_path: Path) -> None:
    got = _drain(OPERATORS[name](tmp_path))
    assert got, name
    if name in EXPECTED:
        assert got == _norm(EXPECTED[name])
    if name in ("shuffle", "shuffle_full"):
        assert sorted(got) == _seq(len(got)) and got != _seq(len(got))
    if name == "sample":
        assert sorted(x for x in got if x < 100) == _seq(6) or sorted(x for x in got if x >= 100) == _seq(9, 100)
    if name == "dynamic_bucket":
        assert all(sum(b) >= 10 for b in got[:-1]) and sum(map(sum, got)) == sum(_seq(12, 1))
    if name == "pack":
        assert all(len(b["seqs"][2]) == 8 for b in got)
    if name == "bucket_by_length":
        assert sum(len(b) for b in got) == 9


@pytest.mark.parametrize("name", sorted(OPERATORS))
def test_operator_state_dict_round_trip(name: str, tmp_path: Path) -> None:
    make = OPERATORS[name]
    want = _drain(make(tmp_path))
    for k in range(len(want) + 1):
        p = make(tmp_path)
        it = iter(p)
        for _ in range(k):
            next(it)
        state = pickle.loads(pickle.dumps(p.state_dict()))       # checkpoints pickle it
        for _ in range(2):
            next(it, None)
        p.load_state_dict(state)
        tail = _drain(p)
        assert tail == want[k:], (name, k)
        q = make(tmp_path)
        q.load_state_dict(state)
        assert _drain(q) == want[k:], (name, k)


@pytest.mark.parametrize("name", sorted(OPERATORS))
def test_operator_reset(name: str, tmp_path: Path) -> None:
    p = OPERATORS[name](tmp_path)
    want = _drain(p)
    p.reset(reset_rng=True)
    assert _drain(p) == want
    it = iter(p)
    p.reset(reset_rng=True)
    next(iter(p))
    p.reset(reset_rng=True)
    assert _drain(p) == want
    del it


# ------------------------------------------------------------------ map(deterministic=False)
def test_unordered_parallel_map_returns_every_element_once() -> None:
    import time

    def slow_for_some(x: int) -> int:
        if x % 7 == 0:
            time.sleep(0.02)
        return x * 2

    p = read_sequence(list(range(100))).map(slow_for_some, num_parallel_calls=4, deterministic=False).and_return()
    out = list(p)
    assert sorted(out) == [2 * i for i in range(100)]
    assert out != sorted(out)                          # the slow elements were overtaken
    p.reset()
    assert sorted(p) == [2 * i for i in range(100)]
    # one call at a time, or deterministic (the default): input order
    assert list(read_sequence(list(range(20))).map(slow_for_some, num_parallel_calls=1, deterministic=False)
                .and_return()) == [2 * i for i in range(20)]
    ordered = read_sequence(list(range(20))).map(slow_for_some, num_parallel_calls=4).and_return()
    assert list(ordered) == [2 * i for i in range(20)]


def test_unordered_parallel_map_position_and_errors() -> None:
    def fn(x: int) -> int:
        return x + 1000

    def build():  # type: ignore[no-untyped-def]
        return read_sequence(list(range(50))).map(fn, num_parallel_calls=3, deterministic=False).and_return()

    p = build()
    it = iter(p)
    head = [next(it) for _ in range(17)]
    state = p.state_dict()
    tail = list(it)
    assert sorted(head + tail) == [i + 1000 for i in range(50)]
    q = build()
    q.load_state_dict(state)
    assert sorted(q) == sorted(tail)                   # what was finished but not handed out is part of the position

    def boom(x: int) -> int:
        if x == 13:
            raise ValueError("thirteen")
        return x

    r = read_sequence(list(range(30))).map(boom, num_parallel_calls=4, deterministic=False).and_return()
    with pytest.raises(Exception, match="thirteen"):
        list(r)
    with pytest.raises(DataPipelineError):
        next(iter(r))                                  # broken until reset
    # native callables run on the workers without the interpreter lock
    from fairseq2_b200.data.text import StrToIntConverter

    s = read_sequence([str(i) for i in range(200)]).map(StrToIntConverter(), num_parallel_calls=8,
                                                         deterministic=False).and_return()
    assert sorted(s) == list(range(200))


# ------------------------------------------------------------------ random operator chains
def _random_chain(rng):  # type: ignore[no-untyped-def]
    chain, bucketed = [], False
    for _ in range(rng.randint(1, 5)):
        k = rng.choice(["map", "pmap", "filter", "shuffle", "bucket", "take", "skip", "prefetch", "shard", "repeat",
                        "unbucket"])
        if bucketed and k in ("map", "pmap", "bucket"):      # the elements are lists now
            k = "unbucket"
        if k == "unbucket" and not bucketed:
            k = "prefetch"
        if k == "pmap":
            chain.append((k, rng.choice([2, 3, 4])))
        elif k == "shuffle":
            chain.append((k, rng.choice([0, 1, 4, 16]), rng.randint(0, 5)))
        elif k == "bucket":
            chain.append((k, rng.choice([1, 2, 5]), rng.random() < 0.5))
            bucketed = True
        elif k == "take":
            chain.append((k, rng.randint(0, 30)))
        elif k == "skip":
            chain.append((k, rng.randint(0, 10)))
        elif k == "prefetch":
            chain.append((k, rng.choice([1, 3])))
        elif k == "shard":
            chain.append((k, rng.randint(0, 1), 2))
        elif k == "repeat":
            chain.append((k, rng.choice([1, 2])))
        else:
            if k == "unbucket":
                bucketed = False
            chain.append((k,))
    return chain


def _build_chain(chain, n: int) -> DataPipeline:  # type: ignore[no-untyped-def]
    b = read_sequence(list(range(n)))
    for op in chain:
        k = op[0]
        if k == "map":
            b = b.map(lambda x: x + 1)
        elif k == "pmap":
            b = b.map(lambda x: x * 2, num_parallel_calls=op[1])
        elif k == "filter":
            b = b.filter(lambda x: (x if isinstance(x, int) else len(x)) % 3 != 0)
        elif k == "shuffle":
            b = b.shuffle(op[1], seed=op[2])
        elif k == "bucket":
            b = b.bucket(op[1], drop_remainder=op[2])
        elif k == "take":
            b = b.take(op[1])
        elif k == "skip":
            b = b.skip(op[1])
        elif k == "prefetch":
            b = b.prefetch(op[1])
        elif k == "shard":
            b = b.shard(op[1], op[2], allow_uneven=True)
        elif k == "repeat":
            b = b.repeat(op[1])
        else:
            b = b.yield_from(lambda xs: read_sequence(list(xs)).and_return())
    return b.and_return()


def test_random_operator_chains_save_and_restore_their_position() -> None:
    """300 random chains of up to five operators: stopping anywhere, saving the position, loading it into a freshly
    built pipeline and reading on gives the uninterrupted output; a reset with the generators rewound does too."""
    import random

    rng = random.Random(0)
    for _ in range(300):
        chain, n = _random_chain(rng), rng.randint(0, 40)
        want = list(_build_chain(chain, n))
        for _ in range(2):
            k = rng.randint(0, len(want))
            p = _build_chain(chain, n)
            it = iter(p)
            head = [next(it) for _ in range(k)]
            state = p.state_dict()
            q = _build_chain(chain, n)
            q.load_state_dict(state)
            assert head + list(q) == want, (chain, n, k)
            p.reset(True)
            assert list(p) == want, (chain, n)
