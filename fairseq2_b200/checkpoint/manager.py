"""Checkpoint manager with the fairseq2 on-disk layout
(cf. ``checkpoint/manager.py:156-873``):

    <dir>/model.yaml
    <dir>/step_N/trainer/rank_RR.pt            every root rank
    <dir>/step_N/model/pp_00/tp_TT/sdp_SS.pt   ranks with rdp.rank == 0 (local shards, FQN keys, pickle protocol 2)
    <dir>/step_N/optimizer/pp_00/tp_TT/sdp_SS.pt
    <dir>/step_N/data_reader/dp_DD.pt          ranks with tp.rank == 0
    <dir>/scores/step_N.txt

A step is written into ``step_N.tmp`` and renamed between two barriers
(two-phase commit). Saving is asynchronous by default: state is first copied to
pinned host memory on a side stream (so the training stream is not blocked by
``.cpu()``), then a background thread serialises it; the commit happens on the
main thread at the next ``maybe_complete_save_operation`` call.
"""
from __future__ import annotations

import shutil
from concurrent.futures import Future
from pathlib import Path
from typing import Any, Callable, Iterable, Mapping

import torch
from torch import Tensor

from fairseq2_b200.error import InvalidOperationError
from fairseq2_b200.gang import Gangs, all_sum
from fairseq2_b200.io import TensorFileDumper, TensorFileError, TensorFileLoader
from fairseq2_b200.logging import log
from fairseq2_b200.utils.threading import StandardThreadPool, ThreadPool


class CheckpointError(Exception):
    pass


class CheckpointNotFoundError(CheckpointError):
    def __init__(self, step_nr: int) -> None:
        super().__init__(f"A checkpoint of step {step_nr} is not found.")
        self.step_nr = step_nr


class CheckpointSaveError(CheckpointError):
    pass


class CheckpointLoadError(CheckpointError):
    pass


def _to_host(obj: Any, stream: "torch.cuda.Stream | None") -> Any:
    """Deep-copies ``obj`` with every CUDA tensor moved to pinned host memory."""
    if isinstance(obj, Tensor):
        if obj.is_cuda:
            host = torch.empty(obj.shape, dtype=obj.dtype, device="cpu", pin_memory=True)
            host.copy_(obj.detach(), non_blocking=True)
            return host
        return obj.detach().clone()
    if isinstance(obj, Mapping):
        return {k: _to_host(v, stream) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        out = [_to_host(v, stream) for v in obj]
        return out if isinstance(obj, list) else tuple(out)
    return obj


class CheckpointManager:
    def __init__(self, checkpoint_dir: Path, gangs: Gangs, *, thread_pool: ThreadPool | None = None,
                 file_loader: TensorFileLoader | None = None, file_dumper: TensorFileDumper | None = None) -> None:
        self._dir = checkpoint_dir
        self._gangs = gangs
        self._pool = thread_pool or StandardThreadPool(1)
        self._loader = file_loader or TensorFileLoader()
        self._dumper = file_dumper or TensorFileDumper()
        self._pending: tuple[int, Future[None], Callable[[int], None] | None] | None = None
        self._copy_stream: torch.cuda.Stream | None = None

    @property
    def checkpoint_dir(self) -> Path:
        return self._dir

    # ------------------------------------------------------------------ save
    def save_checkpoint(self, step_nr: int, trainer: Any, model: Any, optimizer: Any | None, data_reader: Any | None,
                        *, callback: Callable[[int], None] | None = None, blocking: bool = False) -> None:
        """``trainer``/``model``/``optimizer``/``data_reader`` expose ``state_dict()``."""
        self.maybe_complete_save_operation(blocking=True)
        g = self._gangs
        self._begin(step_nr)
        tmp = self._step_dir(step_nr, tmp=True)
        files: list[tuple[Path, Any, int]] = []
        files.append((tmp / f"trainer/rank_{g.root.rank:02d}.pt", trainer.state_dict(), 5))
        pathname = f"pp_{g.pp.rank:02d}/tp_{g.tp.rank:02d}/sdp_{g.sdp.rank:02d}.pt"
        if g.rdp.rank == 0:
            files.append((tmp / "model" / pathname, model.state_dict(), 2))
            if optimizer is not None:
                files.append((tmp / "optimizer" / pathname, optimizer.state_dict(), 5))
        if data_reader is not None and g.tp.rank == 0:
            files.append((tmp / f"data_reader/dp_{g.dp.rank:02d}.pt", data_reader.state_dict(), 5))
        self._do_save(step_nr, files, callback, blocking)

    def save_model_only(self, step_nr: int, model: Any, *, callback: Callable[[int], None] | None = None,
                        blocking: bool = False) -> None:
        self.maybe_complete_save_operation(blocking=True)
        g = self._gangs
        self._begin(step_nr)
        tmp = self._step_dir(step_nr, tmp=True)
        files: list[tuple[Path, Any, int]] = []
        if g.rdp.rank == 0:
            pathname = f"pp_{g.pp.rank:02d}/tp_{g.tp.rank:02d}/sdp_{g.sdp.rank:02d}.pt"
            files.append((tmp / "model" / pathname, model.state_dict(), 2))
        self._do_save(step_nr, files, callback, blocking)

    def _begin(self, step_nr: int) -> None:
        g = self._gangs
        try:
            self.delete_checkpoint(step_nr)
        except CheckpointNotFoundError:
            pass
        if g.root.rank == 0:
            tmp = self._step_dir(step_nr, tmp=True)
            try:
                if tmp.exists():
                    shutil.rmtree(tmp)
                tmp.mkdir(parents=True)
            except OSError as ex:
                raise CheckpointSaveError(f"The temporary directory of step {step_nr} cannot be created: {ex}") from ex
        g.root.barrier()

    def _do_save(self, step_nr: int, files: list[tuple[Path, Any, int]], callback: Callable[[int], None] | None,
                 blocking: bool) -> None:
        dev = self._gangs.root.device
        if dev.type == "cuda":
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(dev)
            self._copy_stream.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(self._copy_stream):
                staged = [(p, _to_host(sd, self._copy_stream), proto) for p, sd, proto in files]
            self._copy_stream.synchronize()
        else:
            staged = [(p, _to_host(sd, None), proto) for p, sd, proto in files]

        def write() -> None:
            for path, sd, proto in staged:
                path.parent.mkdir(parents=True, exist_ok=True)
                self._dumper.dump(sd, path, pickle_protocol=proto)

        if blocking:
            try:
                write()
            except (TensorFileError, OSError) as ex:
                raise CheckpointSaveError(f"The checkpoint of step {step_nr} cannot be saved: {ex}") from ex
            self._commit(step_nr)
            if callback is not None:
                callback(step_nr)
        else:
            self._pending = (step_nr, self._pool.queue(write), callback)

    def maybe_complete_save_operation(self, *, blocking: bool = False) -> bool | None:
        """Returns ``None`` if nothing is pending, else whether the pending save was committed."""
        if self._pending is None:
            return None
        step_nr, fut, callback = self._pending
        g = self._gangs
        if not blocking:
            # all ranks must agree that everyone's write has finished before committing
            done = 1 if fut.done() else 0
            n = int(all_sum(g.root, done).item()) if g.root.size > 1 else done
            if n != g.root.size:
                return False
        try:
            fut.result()
        except (TensorFileError, OSError) as ex:
            self._pending = None
            raise CheckpointSaveError(f"The checkpoint of step {step_nr} cannot be saved: {ex}") from ex
        self._pending = None
        self._commit(step_nr)
        if callback is not None:
            callback(step_nr)
        return True

    def _commit(self, step_nr: int) -> None:
        g = self._gangs
        g.root.barrier()
        if g.root.rank == 0:
            try:
                self._step_dir(step_nr, tmp=True).replace(self._step_dir(step_nr))
            except OSError as ex:
                raise CheckpointSaveError(f"The checkpoint of step {step_nr} cannot be committed: {ex}") from ex
        g.root.barrier()
        log.info("Checkpoint of step {} saved.", step_nr)

    @property
    def is_saving(self) -> bool:
        return self._pending is not None

    # ------------------------------------------------------------------ load
    def _load_file(self, path: Path, step_nr: int) -> dict[str, Any]:
        if not path.exists():
            if not self._step_dir(step_nr).exists():
                raise CheckpointNotFoundError(step_nr)
            raise CheckpointLoadError(f"'{path}' is missing from the checkpoint of step {step_nr}.")
        try:
            return self._loader.load(path, map_location="cpu", restrict=False)
        except TensorFileError as ex:
            raise CheckpointLoadError(f"The checkpoint of step {step_nr} cannot be loaded: {ex}") from ex

    def load_trainer_state(self, step_nr: int, trainer: Any) -> None:
        g = self._gangs
        trainer.load_state_dict(self._load_file(self._step_dir(step_nr) / f"trainer/rank_{g.root.rank:02d}.pt", step_nr))
        g.root.barrier()

    def load_model_state(self, step_nr: int, model: Any) -> None:
        g = self._gangs
        p = self._step_dir(step_nr) / f"model/pp_{g.pp.rank:02d}/tp_{g.tp.rank:02d}/sdp_{g.sdp.rank:02d}.pt"
        model.load_state_dict(self._load_file(p, step_nr))
        g.root.barrier()

    def load_optimizer_state(self, step_nr: int, optimizer: Any) -> None:
        g = self._gangs
        p = self._step_dir(step_nr) / f"optimizer/pp_{g.pp.rank:02d}/tp_{g.tp.rank:02d}/sdp_{g.sdp.rank:02d}.pt"
        optimizer.load_state_dict(self._load_file(p, step_nr))
        g.root.barrier()

    def load_data_reader_state(self, step_nr: int, data_reader: Any) -> None:
        g = self._gangs
        p = self._step_dir(step_nr) / f"data_reader/dp_{g.dp.rank:02d}.pt"
        data_reader.load_state_dict(self._load_file(p, step_nr))
        g.root.barrier()

    # --------------------------------------------------------------- scores
    def save_score(self, step_nr: int, score: float) -> None:
        g = self._gangs
        if g.root.rank == 0:
            d = self._dir / "scores"
            d.mkdir(parents=True, exist_ok=True)
            (d / f"step_{step_nr}.txt").write_text(f"{score}\n")
        g.root.barrier()

    def load_scores(self) -> list[tuple[float, int]]:
        """``(score, step_nr)`` pairs, best score first (cf. reference ``checkpoint/manager.py:527-555``)."""
        out = []
        d = self._dir / "scores"
        if d.exists():
            for f in d.glob("step_*.txt"):
                try:
                    out.append((float(f.read_text().strip()), int(f.stem[5:])))
                except ValueError:
                    raise CheckpointLoadError(f"The score file '{f}' is corrupt.") from None
        out.sort(reverse=True)
        return out

    # --------------------------------------------------------------- listing
    def _step_dir(self, step_nr: int, tmp: bool = False) -> Path:
        return self._dir / (f"step_{step_nr}.tmp" if tmp else f"step_{step_nr}")

    def get_step_numbers(self, *, exclude_model_only: bool = False) -> list[int]:
        steps = []
        if self._dir.exists():
            for d in self._dir.glob("step_*"):
                if not d.is_dir() or d.suffix == ".tmp":
                    continue
                try:
                    n = int(d.name[5:])
                except ValueError:
                    continue
                if exclude_model_only and not (d / "trainer").exists():
                    continue
                steps.append(n)
        steps.sort()
        return steps

    def maybe_get_last_step_number(self, *, exclude_model_only: bool = False) -> int | None:
        s = self.get_step_numbers(exclude_model_only=exclude_model_only)
        return s[-1] if s else None

    def has_checkpoint(self, *, exclude_model_only: bool = False) -> bool:
        return bool(self.get_step_numbers(exclude_model_only=exclude_model_only))

    # -------------------------------------------------------------- deletion
    def delete_checkpoint(self, step_nr: int, *, keep_model: bool = False) -> None:
        g = self._gangs
        d = self._step_dir(step_nr)
        # every rank must see the same answer: look before rank 0 starts deleting, and let rank 0 decide
        from fairseq2_b200.gang import broadcast_flag

        exists = broadcast_flag(g.root, d.exists()) if g.root.size > 1 else d.exists()
        if g.root.rank == 0 and exists:
            try:
                if keep_model:
                    for sub in d.iterdir():
                        if sub.name not in ("model", "hg"):
                            shutil.rmtree(sub) if sub.is_dir() else sub.unlink()
                else:
                    shutil.rmtree(d)
                    sf = self._dir / "scores" / f"step_{step_nr}.txt"
                    if sf.exists():
                        sf.unlink()
            except OSError as ex:
                raise CheckpointError(f"The checkpoint of step {step_nr} cannot be deleted: {ex}") from ex
        g.root.barrier()
        if not exists:
            raise CheckpointNotFoundError(step_nr)

    def get_stale_step_numbers(self, keep_last_n: int | None = None, keep_best_n: int | None = None,
                               keep_every_n_steps: int | None = None) -> list[int]:
        """Step numbers that the retention policy does not keep, ascending (cf. reference
        ``checkpoint/manager.py:754-798``). The last checkpoint is always kept."""
        steps = self.get_step_numbers()
        if not steps or (keep_last_n is None and keep_best_n is None):
            return []
        keep: set[int] = set()
        if keep_last_n is not None:
            keep.update(steps[-keep_last_n:] if keep_last_n > 0 else [])
        if keep_best_n is not None:
            keep.update(s for _, s in self.load_scores()[:keep_best_n])
        if keep_every_n_steps is not None:
            keep.update(s for s in steps if s % keep_every_n_steps == 0)
        keep.add(steps[-1])
        return [s for s in steps if s not in keep]

    def delete_stale_checkpoints(self, *, keep_last_n: int | None = None, keep_best_n: int | None = None,
                                 keep_every_n_steps: int | None = None, keep_model_only: bool = False) -> list[int]:
        """Applies the retention policy; returns the step numbers that were removed."""
        removed = []
        for s in self.get_stale_step_numbers(keep_last_n, keep_best_n, keep_every_n_steps):
            if True:
                try:
                    self.delete_checkpoint(s, keep_model=keep_model_only)
                    removed.append(s)
                except CheckpointNotFoundError:
                    pass
        return removed

    def close(self) -> None:
        self.maybe_complete_save_operation(blocking=True)
        self._pool.close()
