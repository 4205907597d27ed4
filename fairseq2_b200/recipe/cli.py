"""Command line front end of a recipe (cf. fairseq2 ``recipe/cli.py:154-314``):

    python -m recipes.lm.sft OUTPUT_DIR --config-file cfg.yaml --config trainer.max_grad_norm=1.0 ...

Flags: ``--config-file`` (repeatable), ``--config k=v ...``, ``--dump-config``,
``--no-sweep-dir``, ``--checkpoint-dir``, ``--no-rich``, ``--no-exit-on-error``, ``--debug``.
Failures are mapped to exit codes by the registry in ``recipe/exit_codes.py``."""
from __future__ import annotations

import argparse
import sys
import traceback
from pathlib import Path
from typing import Any, Sequence

from fairseq2_b200.logging import configure_logging, log
from fairseq2_b200.recipe.base import Recipe
from fairseq2_b200.recipe.exit_codes import exit_code_for
from fairseq2_b200.recipe.run import load_recipe_config, run_recipe
from fairseq2_b200.utils.config import parse_config_overrides
from fairseq2_b200.utils.structured import unstructure
from fairseq2_b200.utils.yaml import dump_yaml


def _parse(argv: Sequence[str] | None) -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("output_dir", type=Path, nargs="?", help="directory for logs, checkpoints and metrics")
    ap.add_argument("--config-file", dest="config_files", type=Path, action="append", default=[],
                    help="YAML file(s) merged over the default configuration")
    ap.add_argument("--config", dest="overrides", nargs="+", action="extend", default=[], metavar="KEY=VALUE",
                    help="configuration overrides, e.g. optimizer.config.lr=3e-4")
    ap.add_argument("--dump-config", action="store_true", help="print the merged configuration and exit")
    ap.add_argument("--no-sweep-dir", action="store_true", help="do not create a sweep sub-directory")
    ap.add_argument("--checkpoint-dir", type=Path, default=None)
    ap.add_argument("--no-rich", action="store_true",
                    help="plain text console output: no rich formatting, no progress bars")
    ap.add_argument("--no-exit-on-error", action="store_true", help="re-raise errors instead of exiting")
    ap.add_argument("--debug", action="store_true")
    return ap.parse_args(argv)


def main(recipe: Recipe, argv: Sequence[str] | None = None, preset: Any | None = None) -> int:
    args = _parse(argv)
    if args.no_rich:
        import os

        os.environ["FAIRSEQ2_NO_RICH"] = "1"
        os.environ["FAIRSEQ2_NO_PROGRESS"] = "1"
    configure_logging(debug=args.debug, no_rich=args.no_rich)
    try:
        overrides = parse_config_overrides(args.overrides)
        if args.debug:
            overrides.setdefault("common", {})["debug"] = True  # type: ignore[index]
        config = load_recipe_config(recipe, args.config_files, overrides, preset)
        if args.dump_config:
            print(dump_yaml(unstructure(config)), end="")
            return 0
        if args.output_dir is None:
            print("error: OUTPUT_DIR is required unless --dump-config is given", file=sys.stderr)
            return 2
        run_recipe(recipe, config, args.output_dir, checkpoint_dir=args.checkpoint_dir,
                   no_sweep_dir=args.no_sweep_dir or None)
        return 0
    except BaseException as ex:  # noqa: BLE001 - every failure is mapped to an exit code by the registry
        if args.no_exit_on_error and not isinstance(ex, SystemExit):
            raise
        if isinstance(ex, SystemExit):
            raise
        return exit_code_for(ex)
