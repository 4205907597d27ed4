"""Profilers (cf. fairseq2 ``profilers/torch.py:25-77``, ``profilers/composite.py``)."""
from __future__ import annotations

from pathlib import Path
from types import TracebackType
from typing import Sequence

import torch
from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler


class Profiler:
    def start(self) -> None: ...

    def stop(self) -> None: ...

    def step(self) -> None: ...

    def __enter__(self) -> "Profiler":
        self.start()
        return self

    def __exit__(self, et: type[BaseException] | None, ev: BaseException | None, tb: TracebackType | None) -> None:
        self.stop()


class NoopProfiler(Profiler):
    pass


class CompositeProfiler(Profiler):
    def __init__(self, profilers: Sequence[Profiler]) -> None:
        self._ps = list(profilers)

    def start(self) -> None:
        for p in self._ps:
            p.start()

    def stop(self) -> None:
        for p in self._ps:
            p.stop()

    def step(self) -> None:
        for p in self._ps:
            p.step()


class TorchProfiler(Profiler):
    """CPU+CUDA ``torch.profiler`` with a skip/wait/warmup/active schedule; traces go to
    ``<log_dir>/rank_N`` as gzipped TensorBoard traces with shapes, memory, stacks and FLOPs."""

    def __init__(self, skip_n_steps: int, wait_n_steps: int, num_warmup_steps: int, num_active_steps: int,
                 repeat: int, log_dir: Path, rank: int) -> None:
        acts = [ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(ProfilerActivity.CUDA)
        self._prof = profile(
            activities=acts,
            schedule=schedule(skip_first=skip_n_steps, wait=wait_n_steps, warmup=num_warmup_steps,
                              active=num_active_steps, repeat=repeat),
            on_trace_ready=tensorboard_trace_handler(str(log_dir), worker_name=f"rank_{rank}", use_gzip=True),
            record_shapes=True, profile_memory=True, with_stack=True, with_flops=True)

    def start(self) -> None:
        self._prof.start()

    def stop(self) -> None:
        self._prof.stop()

    def step(self) -> None:
        self._prof.step()
