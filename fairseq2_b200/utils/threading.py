"""Background worker pool returning futures (cf. ``src/fairseq2/utils/threading.py``)."""
from __future__ import annotations

import os
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Callable, TypeVar

import torch

T = TypeVar("T")


class ThreadPool:
    def queue(self, fn: Callable[..., T], /, *args: object, **kw: object) -> "Future[T]":
        raise NotImplementedError

    def close(self) -> None: ...


class StandardThreadPool(ThreadPool):
    """Workers run with a capped intra-op thread count so that background
    checkpoint serialization does not oversubscribe the host cores."""

    def __init__(self, max_num_workers: int = 1, num_torch_threads: int | None = None) -> None:
        def init() -> None:
            if num_torch_threads is not None:
                torch.set_num_threads(num_torch_threads)

        self._ex = ThreadPoolExecutor(max_workers=max_num_workers, thread_name_prefix="fs2b200", initializer=init)

    @staticmethod
    def create_default(local_world_size: int) -> "StandardThreadPool":
        n = os.cpu_count() or 1
        return StandardThreadPool(1, max(n // max(local_world_size, 1) // 2, 1))

    def queue(self, fn: Callable[..., T], /, *args: object, **kw: object) -> "Future[T]":
        return self._ex.submit(fn, *args, **kw)

    def close(self) -> None:
        self._ex.shutdown(wait=True)
