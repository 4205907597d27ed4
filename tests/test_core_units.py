"""Unit tests of small core pieces: LR schedulers (closed forms), config merging and directives, structured
conversion, sweep tags, the asset store (environments, base chains), metric bags and the fake gang."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from pathlib import Path

import pytest
import torch

from fairseq2_b200.assets import AssetStore
from fairseq2_b200.assets.card import AssetCardError
from fairseq2_b200.assets.store import AssetMetadataError, AssetNotFoundError, InMemoryAssetMetadataProvider
from fairseq2_b200.metrics import MetricBag
from fairseq2_b200.metrics.aggregation import Max, Mean, Sum
from fairseq2_b200.optim.lr_schedulers import (CosineAnnealingLR, MyleLR, NoamLR, PolynomialDecayLR, TriStageLR,
                                               get_effective_lr)
from fairseq2_b200.recipe.sweep_tag import SweepFormatPlaceholderError, generate_sweep_tag
from fairseq2_b200.utils.config import (merge_config, parse_config_overrides, process_directives,
                                        replace_env_directive, replace_path_directive)
from fairseq2_b200.utils.structured import StructureError, structure, unstructure


def _opt(lr: float = 1.0) -> torch.optim.Optimizer:
    return torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=lr)


def _run(sched, n: int) -> list[float]:  # type: ignore[no-untyped-def]
    out = [get_effective_lr(sched)]
    for _ in range(n):
        sched.optimizer.step()
        sched.step()
        out.append(get_effective_lr(sched))
    return out


def test_cosine_annealing_closed_form() -> None:
    lrs = _run(CosineAnnealingLR(_opt(2.0), cycle_len=10, num_warmup_steps=4, start_lr=0.0, final_lr=0.2), 24)
    assert lrs[:5] == pytest.approx([0.0, 0.5, 1.0, 1.5, 2.0])
    for pos in range(10):
        want = 0.2 + 0.5 * (2.0 - 0.2) * (1 + math.cos(math.pi * pos / 10))
        assert lrs[4 + pos] == pytest.approx(want)
        assert lrs[14 + pos] == pytest.approx(want)             # second cycle repeats with cycle_mul = lr_mul = 1
    grown = _run(CosineAnnealingLR(_opt(1.0), cycle_len=4, num_warmup_steps=0, cycle_mul=2.0, lr_mul=0.5), 12)
    assert grown[0] == pytest.approx(1.0) and grown[4] == pytest.approx(0.5)      # second cycle starts at lr_mul * base
    assert grown[8] == pytest.approx(0.5 * 0.5 * (1 + math.cos(math.pi * 4 / 8)))  # half-way through a cycle of 8
    assert grown[12] == pytest.approx(0.25)


def test_myle_noam_polynomial_tristage() -> None:
    myle = _run(MyleLR(_opt(1.0), num_warmup_steps=4, start_lr=0.2), 16)
    assert myle[0] == pytest.approx(0.2) and myle[4] == pytest.approx(1.0) and myle[16] == pytest.approx(0.5)
    noam = _run(NoamLR(_opt(1.0), num_warmup_steps=4), 16)
    assert noam[0] == 0.0 and noam[2] == pytest.approx(2 * 4 ** -1.5) and noam[16] == pytest.approx(0.25)
    assert max(noam) == pytest.approx(noam[4])
    poly = _run(PolynomialDecayLR(_opt(1.0), num_steps=12, num_warmup_steps=2, power=2.0, final_lr=0.1), 14)
    assert poly[1] == pytest.approx(0.5) and poly[2] == pytest.approx(1.0)
    assert poly[7] == pytest.approx(0.1 + 0.9 * ((12 - 7) / 10) ** 2)
    assert poly[12] == pytest.approx(0.1) and poly[14] == pytest.approx(0.1)
    tri = _run(TriStageLR(_opt(1.0), num_steps=20, stage_ratio=(0.2, 0.3, 0.5), start_lr_scale=0.1, final_lr_scale=0.01), 22)
    assert tri[0] == pytest.approx(0.1) and tri[4] == pytest.approx(1.0) and tri[9] == pytest.approx(1.0)
    assert tri[15] == pytest.approx(math.exp(math.log(0.01) * 5 / 10)) and tri[22] == pytest.approx(0.01)
    with pytest.raises(ValueError):
        TriStageLR(_opt(), num_steps=10, stage_ratio=(0.5, 0.5, 0.5))
    with pytest.raises(ValueError):
        PolynomialDecayLR(_opt(), num_steps=4, num_warmup_steps=4)


def test_merge_config_set_and_del() -> None:
    base = {"a": {"x": 1, "y": {"p": 1, "q": 2}}, "b": [1, 2], "c": 3}
    out = merge_config(base, {"a": {"y": {"q": 5}, "_del_": ["x"]}, "b": [9], "_set_": {"d": {"k": 1}}})
    assert out == {"a": {"y": {"p": 1, "q": 5}}, "b": [9], "c": 3, "d": {"k": 1}}
    assert base["a"]["x"] == 1                                # the base is not modified
    with pytest.raises(TypeError):
        merge_config(base, {"_del_": "x"})


def test_directives_and_overrides(tmp_path: Path) -> None:
    cfg = {"path": "${dir}/data", "user": "${env:WHO}", "fallback": "${env:MISSING:dflt}", "n": 3, "l": ["${env:WHO}"]}
    out = process_directives(cfg, [replace_path_directive(tmp_path), replace_env_directive({"WHO": "me"})])
    assert out == {"path": f"{tmp_path}/data", "user": "me", "fallback": "dflt", "n": 3, "l": ["me"]}
    assert parse_config_overrides(["a.b=1", "a.c=[1, 2]", "d=text", "e=null", "f=true"]) == \
        {"a": {"b": 1, "c": [1, 2]}, "d": "text", "e": None, "f": True}
    with pytest.raises(ValueError):
        parse_config_overrides(["novalue"])


@dataclass
class _Inner:
    rate: float = 0.5
    names: list[str] = field(default_factory=list)


@dataclass
class _Outer:
    inner: _Inner = field(default_factory=_Inner)
    size: int = 1
    path: Path | None = None
    dtype: torch.dtype = torch.float32


def test_structure_round_trip_and_errors() -> None:
    obj = structure({"inner": {"rate": 1, "names": ["a", "b"]}, "size": 4, "path": "/tmp/x", "dtype": "bfloat16"}, _Outer)
    assert obj == _Outer(_Inner(1.0, ["a", "b"]), 4, Path("/tmp/x"), torch.bfloat16)
    un = unstructure(obj)
    assert un == {"inner": {"rate": 1.0, "names": ["a", "b"]}, "size": 4, "path": "/tmp/x", "dtype": "bfloat16"}
    assert structure(un, _Outer) == obj
    with pytest.raises(StructureError, match="size"):
        structure({"size": "many"}, _Outer)
    with pytest.raises(StructureError, match="unknown|extra|nope"):
        structure({"nope": 1}, _Outer)


def test_sweep_tag() -> None:
    cfg = {"model": {"name": "llama3_8b", "flag": True, "none": None}, "optimizer": {"lr": 3e-4},
           "long": "x" * 40, "list": [1, 2]}
    tag = generate_sweep_tag(cfg, 8, "ws_{world_size}.{model.name}.{model.flag}.{model.none}.lr_{optimizer.lr}.{hash}")
    parts = tag.split(".")
    assert parts[0] == "ws_8" and parts[1] == "llama3_8b" and parts[2] == "t" and parts[3] == "none"
    assert tag == generate_sweep_tag(cfg, 8, "ws_{world_size}.{model.name}.{model.flag}.{model.none}.lr_{optimizer.lr}.{hash}")
    other = generate_sweep_tag({**cfg, "optimizer": {"lr": 1e-4}}, 8, "{hash}")
    assert other != generate_sweep_tag(cfg, 8, "{hash}") and len(other) == 8
    assert len(generate_sweep_tag(cfg, 8, "{long}")) == 8                       # long strings are hashed
    with pytest.raises(SweepFormatPlaceholderError):
        generate_sweep_tag(cfg, 8, "{model.nothing}")


def test_asset_store_environments_and_bases() -> None:
    provider = InMemoryAssetMetadataProvider([
        {"name": "base_model", "model_family": "llama", "checkpoint": "https://host/a.pt", "extra": {"k": 1}},
        {"name": "child", "base": "base_model", "checkpoint": "https://host/b.pt"},
        {"name": "child@cluster_x", "checkpoint": "file:///shared/b.pt"},
        {"name": "orphan", "base": "nowhere"},
        {"name": "loop1", "base": "loop2"}, {"name": "loop2", "base": "loop1"},
    ])
    plain = AssetStore([provider])
    card = plain.retrieve_card("child")
    assert card.maybe_get_field("checkpoint", str) == "https://host/b.pt"
    assert card.maybe_get_field("model_family", str) == "llama"                 # falls through to the base card
    on_cluster = AssetStore([provider], env_resolvers=[lambda: "cluster_x"])
    assert on_cluster.retrieve_card("child").maybe_get_field("checkpoint", str) == "file:///shared/b.pt"
    assert on_cluster.retrieve_card("child").maybe_get_field("model_family", str) == "llama"
    assert "child" in plain.retrieve_names() and "child@cluster_x" not in plain.retrieve_names()
    with pytest.raises(AssetNotFoundError):
        plain.retrieve_card("missing")
    with pytest.raises((AssetNotFoundError, AssetMetadataError, AssetCardError)):
        plain.retrieve_card("orphan")
    with pytest.raises(AssetCardError, match="cycle"):
        plain.retrieve_card("loop1")
    with pytest.raises(AssetMetadataError):
        AssetStore([provider, InMemoryAssetMetadataProvider([{"name": "child"}], source="second")]).retrieve_card("child")


def test_metric_bag_updates_rollback_and_state() -> None:
    bag = MetricBag(torch.device("cpu"))
    bag.get("loss", Mean).update(torch.tensor(2.0), weight=2)
    bag.get("total_steps", Sum).update(3)
    bag.begin_updates()
    bag.get("loss", Mean).update(torch.tensor(100.0), weight=1)
    bag.get("peak", Max).update(7)
    bag.rollback_updates()
    assert "peak" not in bag and float(bag.get("loss").compute()) == pytest.approx(2.0)
    bag.begin_updates()
    bag.get("loss", Mean).update(torch.tensor(5.0), weight=1)
    bag.commit_updates()
    assert float(bag.get("loss").compute()) == pytest.approx(3.0)
    state = bag.state_dict()
    assert list(state) == ["total_steps"]                     # only the persistent ("total_") metrics are saved
    bag.reset_non_persistent_metrics()
    assert float(bag.get("total_steps").compute()) == 3.0
    fresh = MetricBag(torch.device("cpu"))
    fresh.get("total_steps", Sum)
    fresh.load_state_dict(state)
    assert float(fresh.get("total_steps").compute()) == 3.0
    with pytest.raises(TypeError):
        bag.get("loss", Sum)


def test_fake_gang_collectives() -> None:
    from fairseq2_b200.gang import FakeGang, ReduceOperation

    g = FakeGang(torch.device("cpu"), rank=1, size=4)
    t = torch.tensor([2.0, 4.0])
    g.all_reduce(t, ReduceOperation.SUM)
    assert t.tolist() == [8.0, 16.0]                          # every fake rank contributes the same value
    t = torch.tensor([2.0])
    g.all_reduce(t, ReduceOperation.MEAN)
    assert t.tolist() == [2.0]
    out = torch.empty(4, 2)
    g.all_gather(out, torch.tensor([1.0, 2.0]))
    assert out.tolist() == [[1.0, 2.0]] * 4
    assert g.broadcast_objects([{"a": 1}], source_rank=0) is None or True
    g.barrier()
