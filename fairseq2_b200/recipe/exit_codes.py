"""Exit-code registry of the recipe command line (cf. fairseq2 ``recipe/cli.py:317-385,526-915``).

Every failure a recipe run can end with is mapped to ONE table row: the exception class (given by its import path,
resolved on first use so that importing the CLI does not import the whole library), the process exit code, the
message that is logged, and whether the stack trace is worth logging. Exceptions are matched along their MRO, so
a subclass inherits the row of its nearest registered base; ``register_cli_error`` adds or replaces rows (the hook
for extensions).

Exit codes: 0 success or requested stop, 1 operational failure (I/O, communication, out of memory, unexpected
errors), 2 the user's configuration or arguments are at fault, 130 interrupted.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Callable

from fairseq2_b200.logging import log

ExceptionHandler = Callable[[BaseException], int]


@dataclass(frozen=True)
class CliErrorRow:
    path: str              # "package.module:ClassName"
    exit_code: int
    message: str           # str.format template; {ex} is the exception, {name} its class name
    trace: bool = False    # log the stack trace as well


# user errors (2): something named in the configuration does not exist or is not valid
_USER = 2
# operational errors (1): the environment failed, not the configuration
_OPER = 1

_ROWS: list[CliErrorRow] = [
    CliErrorRow("fairseq2_b200.recipe.error:RecipeConfigParseError", _USER, "The recipe configuration cannot be parsed: {ex}"),
    CliErrorRow("fairseq2_b200.utils.validation:ValidationError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.utils.structured:StructureError", _USER, "The configuration does not match its schema: {ex}"),
    CliErrorRow("fairseq2_b200.utils.yaml:YamlError", _USER, "A YAML file cannot be read: {ex}"),
    CliErrorRow("fairseq2_b200.recipe.sweep_tag:SweepFormatError", _USER, "`common.sweep_format` is not valid: {ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:ModelNotKnownError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:ModelFamilyNotKnownError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:ModelArchitectureNotKnownError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:ModelCheckpointNotFoundError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:DatasetNotKnownError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:TokenizerNotKnownError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:FSDPNotSupportedError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:GangTopologyError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:DeviceError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:OutputDirectoryError", _OPER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.error:RecipeError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.recipe.component:UnknownComponentError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.models.family:UnknownModelFamilyError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.models.family:UnknownModelArchitectureError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.models.family:ModelFamilyError", _OPER, "The model family failed: {ex}", True),
    CliErrorRow("fairseq2_b200.datasets.family:UnknownDatasetError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.datasets.family:UnknownDatasetFamilyError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.datasets.family:DatasetError", _OPER, "The dataset cannot be opened: {ex}", True),
    CliErrorRow("fairseq2_b200.data.tokenizers.hub:UnknownTokenizerFamilyError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.runtime.config_registry:ConfigNotFoundError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.assets.store:AssetNotFoundError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.assets.store:AssetMetadataError", _OPER, "An asset metadata source is erroneous: {ex}", True),
    CliErrorRow("fairseq2_b200.assets.card:AssetCardError", _OPER, "An asset card is erroneous: {ex}", True),
    CliErrorRow("fairseq2_b200.assets.download_manager:AssetDownloadError", _OPER, "An asset cannot be downloaded: {ex}", True),
    CliErrorRow("fairseq2_b200.checkpoint.manager:CheckpointNotFoundError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.checkpoint.manager:CheckpointError", _OPER, "A checkpoint operation failed: {ex}", True),
    CliErrorRow("fairseq2_b200.model_checkpoint.loader:ModelCheckpointError", _OPER, "The model checkpoint is erroneous: {ex}", True),
    CliErrorRow("fairseq2_b200.io:TensorFileError", _OPER, "A tensor file cannot be read or written: {ex}", True),
    CliErrorRow("fairseq2_b200.datasets.data_reader:DataReadError", _OPER, "{ex}", True),
    CliErrorRow("fairseq2_b200.cluster:ClusterError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.device:DeviceDetectionError", _OPER, "The device of the process cannot be determined: {ex}", True),
    CliErrorRow("fairseq2_b200.utils.env:EnvironmentVariableError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.world_info:InvalidEnvironmentVariableError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.composition.extensions:ExtensionError", _OPER, "An extension failed to initialize: {ex}", True),
    CliErrorRow("fairseq2_b200.trainer:MinimumLossScaleReachedError", _USER,
                "{ex} Lower the learning rate, use bfloat16 or raise `trainer.fp16_loss_scale`."),
    CliErrorRow("fairseq2_b200.trainer:InconsistentGradNormError", _OPER,
                "{ex} The replicas have diverged; check the logs of every rank.", True),
    CliErrorRow("fairseq2_b200.ops._ext:KernelWaitTimeout", _OPER,
                "{ex} A peer process did not reach a collective in time; check the logs of the other ranks.", True),
    CliErrorRow("fairseq2_b200.gang:GangError", _OPER, "A collective operation failed: {ex}", True),
    CliErrorRow("fairseq2_b200.error:OperationalError", _OPER, "The recipe failed due to an operational error: {ex}", True),
    CliErrorRow("fairseq2_b200.error:NotSupportedError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.error:StateDictError", _OPER, "A state dictionary does not fit its target: {ex}", True),
    CliErrorRow("fairseq2_b200.sharder:ShardSpecError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.models.utils.hg_export:HuggingFaceExportError", _OPER, "The Hugging Face export failed: {ex}", True),
    CliErrorRow("fairseq2_b200.models.hg.adapter:HuggingFaceModelError", _USER, "{ex}"),
    CliErrorRow("fairseq2_b200.utils.process:ProcessError", _OPER, "A child process failed: {ex}", True),
    CliErrorRow("fairseq2_b200.runtime.dependency:DependencyError", _OPER, "The object graph cannot be built: {ex}", True),
    CliErrorRow("fairseq2_b200.error:InternalError", _OPER, "Internal error, please file a bug report: {ex}", True),
    CliErrorRow("torch:OutOfMemoryError", _OPER, "The device ran out of memory: {ex}", True),
    CliErrorRow("builtins:FileNotFoundError", _USER, "{ex}"),
    CliErrorRow("builtins:PermissionError", _OPER, "{ex}"),
    CliErrorRow("builtins:ValueError", _USER, "{ex}"),
]

_custom: dict[type, ExceptionHandler] = {}
_resolved: dict[type, CliErrorRow] | None = None


def register_cli_error(kls: type[BaseException], handler: ExceptionHandler) -> None:
    """``handler(ex) -> exit code`` takes precedence over the built-in table for ``kls`` and its subclasses."""
    _custom[kls] = handler


def _table() -> dict[type, CliErrorRow]:
    global _resolved
    if _resolved is None:
        _resolved = {}
        for row in _ROWS:
            mod, _, name = row.path.partition(":")
            try:
                kls = getattr(importlib.import_module(mod), name)
            except (ImportError, AttributeError):
                continue            # an optional part of the library that is not installed
            _resolved.setdefault(kls, row)
    return _resolved


def registered_cli_errors() -> dict[type, CliErrorRow]:
    """The built-in table, resolved to classes (for documentation and tests)."""
    return dict(_table())


def exit_code_for(ex: BaseException) -> int:
    """Logs the failure the way its row says and returns the exit code of the process."""
    from fairseq2_b200.task import TaskStopException

    if isinstance(ex, TaskStopException):
        return 0
    if isinstance(ex, KeyboardInterrupt):
        return 130
    for kls in type(ex).__mro__:
        handler = _custom.get(kls)
        if handler is not None:
            return handler(ex)
        row = _table().get(kls)
        if row is not None:
            msg = row.message.format(ex=ex, name=type(ex).__name__)
            if row.trace or ex.__cause__ is not None:
                log.exception("{}", msg, exc_info=ex)
            else:
                log.error("{}", msg)
            return row.exit_code
    log.exception("The recipe failed due to an unexpected error ({}). Please file a bug report.", type(ex).__name__,
                  exc_info=ex)
    return 1
