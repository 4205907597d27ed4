"""Validation tree walk, URIs, environment helpers, early stopper protocol, stopwatch and RNG bag."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path

import pytest
import torch

from fairseq2_b200.utils.env import Environment, EnvironmentVariableError, get_int, get_path, get_rank, get_world_size
from fairseq2_b200.utils.rng import RngBag, temporary_manual_seed
from fairseq2_b200.utils.stopwatch import Stopwatch
from fairseq2_b200.utils.uri import Uri
from fairseq2_b200.utils.validation import ValidationError, ValidationResult, validate


@dataclass
class _Leaf:
    rate: float = 0.5

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        if not 0.0 <= self.rate <= 1.0:
            r.add_error(f"`rate` must be in [0, 1], but is {self.rate} instead.")
        return r


@dataclass
class _Root:
    leaf: _Leaf = field(default_factory=_Leaf)
    leaves: list[_Leaf] = field(default_factory=list)
    size: int = 1

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        if self.size < 1:
            r.add_error("`size` must be positive.")
        return r


def test_validation_walks_nested_objects() -> None:
    validate(_Root())
    with pytest.raises(ValidationError) as info:
        validate(_Root(leaf=_Leaf(2.0), leaves=[_Leaf(0.1), _Leaf(-1.0)], size=0))
    msg = str(info.value)
    assert "size" in msg and "leaf" in msg and "leaves" in msg and msg.count("rate") >= 2


def test_uri() -> None:
    u = Uri.maybe_parse("https://host.example/a/b.pt")
    assert u is not None and u.scheme == "https" and str(u) == "https://host.example/a/b.pt"
    f = Uri.maybe_parse("file:///tmp/x.pt")
    assert f is not None and f.scheme == "file" and f.to_path() == Path("/tmp/x.pt")
    assert Uri.maybe_parse("/plain/path") is None and Uri.maybe_parse("relative/path.pt") is None
    hg = Uri.maybe_parse("hg://org/repo")
    assert hg is not None and hg.scheme == "hg"


def test_environment_helpers() -> None:
    env = Environment({"RANK": "3", "WORLD_SIZE": "8", "BAD": "x", "HOME_DIR": "~/data"})
    assert get_rank(env) == 3 and get_world_size(env) == 8 and get_int(env, "MISSING", 7) == 7
    assert get_path(env, "HOME_DIR") == Path("~/data").expanduser() and get_path(env, "MISSING") is None
    with pytest.raises(EnvironmentVariableError):
        get_int(env, "BAD")
    env.set("NEW", "1")
    assert env.has("NEW") and env.maybe_get("NOPE") is None and "NEW" in env.to_dict()


def test_stopwatch_accumulates_between_start_and_stop() -> None:
    sw = Stopwatch()
    assert sw.get_elapsed_time() == 0.0
    sw.start()
    time.sleep(0.02)
    sw.stop()
    first = sw.get_elapsed_time()
    assert first >= 0.02
    time.sleep(0.02)
    assert sw.get_elapsed_time() == first                      # stopped: no time passes
    sw.start()
    time.sleep(0.01)
    sw.stop()
    assert sw.get_elapsed_time() > first
    sw.reset()
    assert sw.get_elapsed_time() == 0.0
    with pytest.raises(RuntimeError):
        sw.start()
        sw.start()


def test_rng_bag_state_round_trip_and_temporary_seed() -> None:
    bag = RngBag.from_device_defaults(torch.device("cpu"))
    bag.manual_seed(5)
    state = bag.state_dict()
    a = torch.rand(3)
    bag.load_state_dict(state)
    assert torch.equal(torch.rand(3), a)
    torch.manual_seed(1)
    before = torch.rand(1)
    torch.manual_seed(1)
    with temporary_manual_seed(99, torch.device("cpu")):
        torch.rand(10)                                         # consumes the temporary generator state only
    assert torch.equal(torch.rand(1), before)
