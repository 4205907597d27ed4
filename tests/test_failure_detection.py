"""Failure detection exercised on the host: every failure is made by a CPU process (a rank that raises or exits,
a signal, a file that is missing or damaged); nothing here touches a GPU.

* a gloo rank that dies before a collective -> the surviving rank gets ``GangError`` within the gang's timeout;
* ``SIGUSR1`` in the middle of a run -> the trainer finishes the step, writes a checkpoint and stops with
  ``TaskStopException``; the run resumes from that checkpoint;
* a checkpoint whose shard file is missing, or is not a tensor file -> ``CheckpointLoadError`` on resume.
"""
from __future__ import annotations

import os
import signal
import time
from datetime import timedelta
from pathlib import Path

import pytest
import torch

from tests.dist_utils import run_distributed
from tests.test_trainer import _make


def _dying_rank_worker(rank: int, world: int, mode: str):
    from fairseq2_b200.gang import GangError, ProcessGroupGang, ReduceOperation

    gang = ProcessGroupGang.create_default_process_group(torch.device("cpu"), timeout=timedelta(seconds=8))
    t = torch.ones(4)
    gang.all_reduce(t, ReduceOperation.SUM)          # everyone is alive here
    assert float(t[0]) == world
    if rank == 1:
        if mode == "exit":
            os._exit(0)                              # the process is gone without a goodbye
        return "raised"                              # an exception path: the rank simply never joins again
    t0 = time.monotonic()
    try:
        gang.all_reduce(t, ReduceOperation.SUM)
        gang.barrier()
    except GangError as ex:
        return ("gang_error", time.monotonic() - t0, str(ex)[:80])
    return ("no_error", time.monotonic() - t0, "")


@pytest.mark.parametrize("mode", ["exit", "raise"])
def test_surviving_rank_gets_gang_error_within_the_timeout(mode: str) -> None:
    import torch.multiprocessing as mp

    from tests.dist_utils import _entry, _free_port

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, 2, port, _dying_rank_worker, (mode,), out)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    deadline = time.monotonic() + 90
    while 0 not in got and time.monotonic() < deadline:
        try:
            rank, status, payload = out.get(timeout=5)
            got[rank] = (status, payload)
        except Exception:  # noqa: BLE001 - queue.Empty
            pass
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    assert 0 in got, "the surviving rank never returned"
    status, payload = got[0]
    assert status == "ok", payload
    kind, seconds, _ = payload
    assert kind == "gang_error"
    assert seconds < 60.0


def test_sigusr1_checkpoints_and_stops_then_resumes(tmp_path: Path) -> None:
    from fairseq2_b200.task import TaskStopException
    from fairseq2_b200.trainer import install_stop_signal_handler

    losses: list[float] = []
    trainer, ckpt = _make(tmp_path, losses, max_steps=10, ckpt_every=100)
    old = signal.getsignal(signal.SIGUSR1)
    try:
        install_stop_signal_handler(trainer)
        unit = trainer._unit
        orig = unit.process_batch

        def process_batch(batch, metric_bag=None):
            if len(losses) == 2:                                   # in the middle of the third step
                os.kill(os.getpid(), signal.SIGUSR1)
            return orig(batch, metric_bag)

        unit.process_batch = process_batch
        with pytest.raises(TaskStopException):
            trainer.run()
    finally:
        signal.signal(signal.SIGUSR1, old)
        trainer.close()
    assert trainer.step_nr == 3                                    # the interrupted step was completed
    assert ckpt.get_step_numbers() == [3]                          # and a full checkpoint written on the way out
    more: list[float] = []
    resumed, _ = _make(tmp_path, more, max_steps=5, ckpt_every=100)
    resumed.run()
    resumed.close()
    assert resumed.step_nr == 5 and len(more) == 2


@pytest.mark.parametrize("damage", ["missing_model", "corrupt_optimizer", "missing_trainer"])
def test_resume_from_damaged_checkpoint_raises_typed_error(tmp_path: Path, damage: str) -> None:
    from fairseq2_b200.checkpoint.manager import CheckpointLoadError

    t, ckpt = _make(tmp_path, [], max_steps=2, ckpt_every=2)
    t.run()
    t.close()
    step = tmp_path / "checkpoints" / "step_2"
    if damage == "missing_model":
        (step / "model" / "pp_00" / "tp_00" / "sdp_00.pt").unlink()
    elif damage == "corrupt_optimizer":
        (step / "optimizer" / "pp_00" / "tp_00" / "sdp_00.pt").write_bytes(b"this is not a tensor file")
    else:
        (step / "trainer" / "rank_00.pt").write_bytes(b"\x00" * 16)
    t2, _ = _make(tmp_path, [], max_steps=4, ckpt_every=2)
    with pytest.raises(CheckpointLoadError):
        t2.run()
    t2.close()


def test_missing_data_reader_state_is_an_error_not_a_silent_restart(tmp_path: Path) -> None:
    from fairseq2_b200.checkpoint.manager import CheckpointLoadError

    t, _ = _make(tmp_path, [], max_steps=2, ckpt_every=2)
    t.run()
    t.close()
    (tmp_path / "checkpoints" / "step_2" / "data_reader" / "dp_00.pt").unlink()
    t2, _ = _make(tmp_path, [], max_steps=4, ckpt_every=2)
    with pytest.raises(CheckpointLoadError):
        t2.run()
    t2.close()
