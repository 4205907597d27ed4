"""The command line maps every known failure to an exit code through one registry."""
from __future__ import annotations

import pytest

from fairseq2_b200.recipe.exit_codes import exit_code_for, register_cli_error, registered_cli_errors


def test_table_resolves_and_is_large_enough() -> None:
    table = registered_cli_errors()
    assert len(table) >= 50
    assert all(row.exit_code in (1, 2) for row in table.values())


def test_exit_codes_follow_the_mro() -> None:
    from fairseq2_b200.checkpoint.manager import CheckpointLoadError, CheckpointNotFoundError
    from fairseq2_b200.gang import GangError
    from fairseq2_b200.ops._ext import KernelWaitTimeout
    from fairseq2_b200.recipe.error import ModelNotKnownError
    from fairseq2_b200.task import TaskStopException
    from fairseq2_b200.trainer import MinimumLossScaleReachedError

    assert exit_code_for(ModelNotKnownError("foo")) == 2
    assert exit_code_for(CheckpointNotFoundError(3)) == 2
    assert exit_code_for(CheckpointLoadError("x")) == 1          # inherits the CheckpointError row
    assert exit_code_for(GangError("peer died")) == 1
    assert exit_code_for(KernelWaitTimeout(1, 18)) == 1
    assert exit_code_for(MinimumLossScaleReachedError(7)) == 2
    assert exit_code_for(TaskStopException()) == 0
    assert exit_code_for(KeyboardInterrupt()) == 130
    assert exit_code_for(ZeroDivisionError()) == 1               # unknown: unexpected error


def test_extensions_can_register_handlers() -> None:
    class MyError(Exception):
        pass

    register_cli_error(MyError, lambda ex: 42)
    assert exit_code_for(MyError()) == 42


def test_cli_flags(capsys: pytest.CaptureFixture[str]) -> None:
    from fairseq2_b200.recipe.cli import main
    from recipes.lm.sft.recipe import LMSFTRecipe

    assert main(LMSFTRecipe(), ["--dump-config", "--no-rich"]) == 0
    assert "trainer" in capsys.readouterr().out
    assert main(LMSFTRecipe(), ["--dump-config", "--config", "model.name=does_not_exist_anywhere", "--no-rich"]) in (0, 2)
    assert main(LMSFTRecipe(), ["--no-rich"]) == 2               # OUTPUT_DIR missing
