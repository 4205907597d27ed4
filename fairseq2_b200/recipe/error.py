"""Typed recipe errors mapped to CLI exit codes (cf. fairseq2 ``recipe/error.py``)."""
from __future__ import annotations


class RecipeError(Exception):
    exit_code = 1


class RecipeConfigParseError(RecipeError):
    exit_code = 2


class ModelNotKnownError(RecipeError):
    exit_code = 3

    def __init__(self, name: str) -> None:
        super().__init__(f"'{name}' is not a known model.")
        self.name = name


class ModelFamilyNotKnownError(RecipeError):
    exit_code = 3


class ModelArchitectureNotKnownError(RecipeError):
    exit_code = 3


class ModelCheckpointNotFoundError(RecipeError):
    exit_code = 4


class DatasetNotKnownError(RecipeError):
    exit_code = 5


class TokenizerNotKnownError(RecipeError):
    exit_code = 6


class FSDPNotSupportedError(RecipeError):
    exit_code = 7

    def __init__(self) -> None:
        super().__init__("The model family does not support FSDP.")


class MinimumLossScaleReachedExit(RecipeError):
    exit_code = 8


class InconsistentGradNormExit(RecipeError):
    exit_code = 9


class OutputDirectoryError(RecipeError):
    exit_code = 10


class DeviceError(RecipeError):
    exit_code = 11


class GangTopologyError(RecipeError):
    exit_code = 12

    def __init__(self, world_size: int, tp_size: int) -> None:
        super().__init__(f"The number of processes ({world_size}) must be a multiple of `gang.tensor_parallel_size` ({tp_size}).")
