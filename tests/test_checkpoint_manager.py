"""Checkpoint directory layout, two-phase commit, scores and the retention policies
(cf. fairseq2 ``checkpoint/manager.py``: layout :275-387, policies :754-798)."""
from __future__ import annotations

from pathlib import Path

import pytest
import torch

from fairseq2_b200.checkpoint import CheckpointManager
from fairseq2_b200.checkpoint.manager import CheckpointNotFoundError
from fairseq2_b200.gang import FakeGang, Gangs


class _Stateful:
    def __init__(self, **state):  # type: ignore[no-untyped-def]
        self.state = dict(state)

    def state_dict(self):  # type: ignore[no-untyped-def]
        return dict(self.state)

    def load_state_dict(self, sd):  # type: ignore[no-untyped-def]
        self.state = dict(sd)


def _gangs() -> Gangs:
    g = FakeGang(torch.device("cpu"))
    return Gangs(root=g, dp=g, rdp=g, sdp=g, tp=g, pp=g)


def _save(m: CheckpointManager, step: int, score: float | None = None) -> None:
    m.save_checkpoint(step, _Stateful(step_nr=step), _Stateful(w=torch.full((2,), float(step))), _Stateful(lr=0.1),
                      _Stateful(pos=step * 10), blocking=True)
    if score is not None:
        m.save_score(step, score)


def test_layout_and_reload(tmp_path: Path) -> None:
    m = CheckpointManager(tmp_path / "checkpoints", _gangs())
    _save(m, 10)
    step = tmp_path / "checkpoints" / "step_10"
    assert (step / "trainer" / "rank_00.pt").is_file()
    assert (step / "model" / "pp_00" / "tp_00" / "sdp_00.pt").is_file()
    assert (step / "optimizer" / "pp_00" / "tp_00" / "sdp_00.pt").is_file()
    assert (step / "data_reader" / "dp_00.pt").is_file()
    assert not (tmp_path / "checkpoints" / "step_10.tmp").exists()              # committed by rename
    sd = torch.load(step / "model" / "pp_00" / "tp_00" / "sdp_00.pt", weights_only=True)
    assert sd["w"].tolist() == [10.0, 10.0]
    model, trainer, reader = _Stateful(), _Stateful(), _Stateful()
    m.load_model_state(10, model)
    m.load_trainer_state(10, trainer)
    m.load_data_reader_state(10, reader)
    assert model.state["w"].tolist() == [10.0, 10.0] and trainer.state["step_nr"] == 10 and reader.state["pos"] == 100
    with pytest.raises(CheckpointNotFoundError):
        m.load_model_state(11, model)
    m.close()


def test_model_only_checkpoints_are_not_resume_points(tmp_path: Path) -> None:
    m = CheckpointManager(tmp_path, _gangs())
    _save(m, 5)
    m.save_model_only(8, _Stateful(w=torch.zeros(1)), blocking=True)
    assert m.get_step_numbers() == [5, 8]
    assert m.get_step_numbers(exclude_model_only=True) == [5]
    assert m.maybe_get_last_step_number(exclude_model_only=True) == 5 and m.maybe_get_last_step_number() == 8
    m.close()


def test_retention_policies(tmp_path: Path) -> None:
    m = CheckpointManager(tmp_path, _gangs())
    for step, score in ((10, 0.3), (20, 0.9), (30, 0.5), (40, 0.1), (50, 0.2)):
        _save(m, step, score)
    assert (tmp_path / "scores" / "step_20.txt").read_text().strip().startswith("0.9")
    assert sorted(m.load_scores(), reverse=True)[0] == (0.9, 20)
    removed = m.delete_stale_checkpoints(keep_last_n=1, keep_best_n=2)
    assert sorted(removed) == [10, 40] and m.get_step_numbers() == [20, 30, 50]   # two best + the last one
    _save(m, 60, 0.05)
    _save(m, 70, 0.01)
    removed = m.delete_stale_checkpoints(keep_last_n=2, keep_every_n_steps=30)
    assert m.get_step_numbers() == [30, 60, 70] and sorted(removed) == [20, 50]
    assert m.delete_stale_checkpoints() == []
    m.delete_checkpoint(30)
    with pytest.raises(CheckpointNotFoundError):
        m.delete_checkpoint(30)
    m.close()
