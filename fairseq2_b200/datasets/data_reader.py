"""Data readers (cf. fairseq2 ``datasets/data_reader.py:24-200``): iterate over
lists of ``num_accumulate`` batches and keep data-parallel ranks in step.

``SyncMode.UNTIL_FIRST`` stops all ranks when the first one runs out of data
(the default for training), ``UNTIL_LAST`` keeps going with empty lists until
the last one finishes (evaluation). The per-step count exchange runs on a CPU
(gloo) side gang when one is given so the hot loop never blocks on a device
read-back."""
from __future__ import annotations

from abc import ABC, abstractmethod
from enum import Enum
from typing import Any, Generic, Iterator, Mapping, Sequence, TypeVar

import torch

from fairseq2_b200.gang import Gang, ReduceOperation

BatchT = TypeVar("BatchT")


class SyncMode(Enum):
    UNTIL_FIRST = 0
    UNTIL_LAST = 1


class DataReadError(Exception):
    pass


class DataReader(ABC, Generic[BatchT]):
    @abstractmethod
    def __iter__(self) -> "DataReader[BatchT]": ...

    @abstractmethod
    def __next__(self) -> list[BatchT]: ...

    @abstractmethod
    def reset(self) -> None: ...

    @abstractmethod
    def state_dict(self) -> dict[str, Any]: ...

    @abstractmethod
    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None: ...

    @property
    @abstractmethod
    def dataset_name(self) -> str: ...

    @property
    @abstractmethod
    def num_accumulate(self) -> int: ...


class DataPipelineReader(DataReader[BatchT]):
    """Reads batches from a data pipeline (anything iterable with
    ``reset()``/``state_dict()``/``load_state_dict()``)."""

    def __init__(self, name: str, split: str, pipeline: Any, gang: Gang, *, num_accumulate: int = 1,
                 drop_remainder: bool = True, sync: bool = True, sync_mode: SyncMode = SyncMode.UNTIL_FIRST,
                 sync_gang: Gang | None = None, strict_state: bool = True) -> None:
        self._name, self._split, self._pipeline, self._gang = name, split, pipeline, gang
        self._num_accumulate = num_accumulate
        self._drop_remainder, self._sync, self._sync_mode = drop_remainder, sync, sync_mode
        self._sync_gang = sync_gang or gang
        self._strict_state = strict_state
        self._iter: Iterator[BatchT] | None = None
        self._eod = False

    def __iter__(self) -> "DataPipelineReader[BatchT]":
        return self

    def __next__(self) -> list[BatchT]:
        if self._eod:
            raise StopIteration()
        if self._iter is None:
            self._iter = iter(self._pipeline)
        batches: list[BatchT] = []
        for _ in range(self._num_accumulate):
            try:
                batches.append(next(self._iter))
            except StopIteration:
                break
            except Exception as ex:  # noqa: BLE001
                raise DataReadError(f"The '{self._split}' split of '{self._name}' cannot be read: {ex}") from ex
        if self._drop_remainder and len(batches) != self._num_accumulate:
            batches = []
        local = len(batches)
        if self._sync and self._sync_gang.size > 1:
            g = self._sync_gang
            t = torch.tensor([local], dtype=torch.int64, device=g.device)
            if self._sync_mode == SyncMode.UNTIL_FIRST:
                g.all_reduce(t, ReduceOperation.MIN)
                n = int(t)
                batches = batches[:n]
                if n == 0:
                    self._eod = True
            else:
                g.all_reduce(t, ReduceOperation.MAX)
                if int(t) == 0:
                    self._eod = True
        elif local == 0:
            self._eod = True
        if self._eod:
            raise StopIteration()
        return batches

    def reset(self) -> None:
        self._eod = False
        self._iter = None
        self._pipeline.reset()

    @property
    def stateless(self) -> bool:
        """True if the underlying pipeline cannot record its position (no ``load_state_dict``)."""
        return not hasattr(self._pipeline, "load_state_dict")

    def state_dict(self) -> dict[str, Any]:
        if self.stateless:
            return {}
        try:
            return self._pipeline.state_dict(strict=self._strict_state)
        except TypeError:
            return self._pipeline.state_dict()

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        self._eod = False
        self._iter = None
        self._pipeline.load_state_dict(state_dict)

    @property
    def dataset_name(self) -> str:
        return self._name

    @property
    def split(self) -> str:
        return self._split

    @property
    def num_accumulate(self) -> int:
        return self._num_accumulate
