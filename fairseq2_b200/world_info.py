"""Rank/size of this process as set by torchrun or Slurm (cf. ``src/fairseq2/world_info.py``)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Mapping


class InvalidEnvironmentVariableError(Exception):
    def __init__(self, var_name: str, message: str) -> None:
        super().__init__(message)
        self.var_name = var_name


def _int_env(env: Mapping[str, str], name: str, default: int, *, minimum: int) -> int:
    s = env.get(name)
    if s is None:
        return default
    try:
        v = int(s)
    except ValueError:
        raise InvalidEnvironmentVariableError(
            name, f"`{name}` environment variable is expected to be an integer, but is '{s}' instead.") from None
    if v < minimum:
        raise InvalidEnvironmentVariableError(
            name, f"`{name}` environment variable must be >= {minimum}, but is {v} instead.")
    return v


@dataclass(frozen=True)
class WorldInfo:
    rank: int = 0
    size: int = 1
    local_rank: int = 0
    local_size: int = 1

    def __post_init__(self) -> None:
        if not 0 <= self.rank < self.size:
            raise ValueError(f"`rank` must be in [0, {self.size}), but is {self.rank} instead.")
        if not 0 <= self.local_rank < self.local_size:
            raise ValueError(f"`local_rank` must be in [0, {self.local_size}), but is {self.local_rank} instead.")

    @staticmethod
    def from_env(env: Mapping[str, str] | None = None) -> "WorldInfo":
        env = os.environ if env is None else env
        size = _int_env(env, "WORLD_SIZE", 1, minimum=1)
        rank = _int_env(env, "RANK", 0, minimum=0)
        local_size = _int_env(env, "LOCAL_WORLD_SIZE", 1, minimum=1)
        local_rank = _int_env(env, "LOCAL_RANK", 0, minimum=0)
        if rank >= size:
            raise InvalidEnvironmentVariableError("RANK", f"`RANK` must be less than `WORLD_SIZE` ({size}), but is {rank}.")
        if local_rank >= local_size:
            raise InvalidEnvironmentVariableError(
                "LOCAL_RANK", f"`LOCAL_RANK` must be less than `LOCAL_WORLD_SIZE` ({local_size}), but is {local_rank}.")
        return WorldInfo(rank, size, local_rank, local_size)
