"""Metric recorders: JSONL files per category, composite fan-out, descriptors and formatting
(cf. fairseq2 ``metrics/recorders/jsonl.py:52-103``, ``descriptor.py``, ``formatters.py``)."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from fairseq2_b200.metrics.recorders.recorder import (CompositeMetricRecorder, JsonlMetricRecorder, MetricRecorder,
                                                      format_metric_value, get_metric_descriptor)


class _Spy(MetricRecorder):
    def __init__(self) -> None:
        self.calls: list[tuple[str, dict, int | None]] = []
        self.closed = False

    def record_metric_values(self, category, values, step_nr=None):  # type: ignore[no-untyped-def]
        self.calls.append((category, dict(values), step_nr))

    def close(self) -> None:
        self.closed = True


def test_jsonl_recorder_writes_one_file_per_category(tmp_path: Path) -> None:
    rec = JsonlMetricRecorder(tmp_path)
    rec.record_metric_values("train", {"nll_loss": torch.tensor(1.5), "num_examples": 8, "lr": 1e-4}, step_nr=10)
    rec.record_metric_values("train", {"nll_loss": 1.25, "num_examples": 8}, step_nr=20)
    rec.record_metric_values("valid/dev", {"nll_loss": 2.0}, step_nr=20)
    rec.close()
    train = [json.loads(line) for line in (tmp_path / "train.jsonl").read_text().splitlines()]
    assert [r["Step"] for r in train] == [10, 20] and all("Time" in r for r in train)
    loss_key = get_metric_descriptor("nll_loss").display_name          # values are keyed by their display names
    lr_key = get_metric_descriptor("lr").display_name if get_metric_descriptor("lr") else "lr"
    assert train[0][loss_key] == 1.5 and train[1][loss_key] == 1.25 and train[0][lr_key] == 1e-4
    valid = list(tmp_path.rglob("*.jsonl"))
    assert len(valid) == 2                                     # the slash in the category becomes a safe file name


def test_composite_recorder_fans_out_and_closes() -> None:
    a, b = _Spy(), _Spy()
    comp = CompositeMetricRecorder([a, b])
    comp.record_metric_values("train", {"x": 1}, 3)
    comp.close()
    assert a.calls == b.calls == [("train", {"x": 1}, 3)] and a.closed and b.closed


def test_descriptors_and_formatting() -> None:
    d = get_metric_descriptor("nll_loss")
    assert d is not None and d.display_name and d.higher_better is False
    assert get_metric_descriptor("no_such_metric") is None
    assert format_metric_value("num_examples", 12345) == "12,345"
    assert format_metric_value("wall_time", 3.0).endswith("s")
    assert "%" in format_metric_value("padding_ratio", 0.25)
    assert isinstance(format_metric_value("something_unknown", 1.23456789), str)
