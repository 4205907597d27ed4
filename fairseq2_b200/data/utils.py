"""Helpers for plain Python iterators inside a ``DataPipeline`` (cf. fairseq2 ``data/utils.py:13-62``)."""
from __future__ import annotations

from typing import Callable, Generic, Iterator, TypeVar

from fairseq2_b200.data.data_pipeline import DataPipelineBuilder, read_iterator

T = TypeVar("T")


class IteratorPickleWrapper(Generic[T]):
    """Makes an iterator picklable (and hence checkpointable by ``read_iterator``) by remembering how many items it
    has yielded: unpickling builds a fresh iterator from the factory and skips that many."""

    def __init__(self, iterator_factory: Callable[[], Iterator[T]]) -> None:
        self._factory = iterator_factory
        self._iterator = iterator_factory()
        self._counter = 0

    def __iter__(self) -> "IteratorPickleWrapper[T]":
        return self

    def __next__(self) -> T:
        item = next(self._iterator)
        self._counter += 1
        return item

    def __getstate__(self) -> tuple[Callable[[], Iterator[T]], int]:
        return self._factory, self._counter

    def __setstate__(self, state: tuple[Callable[[], Iterator[T]], int]) -> None:
        self._factory, counter = state
        self._iterator = self._factory()
        for _ in range(counter):
            next(self._iterator)
        self._counter = counter


def read_pickle_wrapped_iterator(iterator_factory: Callable[[], Iterator[T]]) -> DataPipelineBuilder:
    """``read_iterator`` over a generator or other unpicklable iterator; its position survives ``state_dict``."""
    return read_iterator(IteratorPickleWrapper(iterator_factory), reset_fn=lambda it: IteratorPickleWrapper(iterator_factory),
                         infinite=False)
