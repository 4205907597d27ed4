"""Runs a recipe end to end (cf. fairseq2 ``recipe/run.py:76-235``,
``recipe/cli.py:154-482``): load + merge + validate the config, prepare the
cluster environment, per-rank log files, dump ``config.yaml``, configure torch
(seeds, threads, TF32, default SDPA), build the task and run it with graceful
stop on SIGUSR1."""
from __future__ import annotations

import os
import random
from pathlib import Path
from typing import Any, Mapping, Sequence

import numpy as np
import torch

from fairseq2_b200.cluster import prepare_cluster
from fairseq2_b200.logging import configure_logging, log
from fairseq2_b200.recipe.base import Recipe, RecipeContext
from fairseq2_b200.recipe.config import CommonSection
from fairseq2_b200.recipe.error import RecipeConfigParseError
from fairseq2_b200.recipe.sweep_tag import generate_sweep_tag
from fairseq2_b200.task import TaskStopException
from fairseq2_b200.trainer import install_stop_signal_handler
from fairseq2_b200.utils.config import (merge_config, process_directives, replace_env_directive,
                                        replace_path_directive)
from fairseq2_b200.utils.structured import StructureError, structure, unstructure
from fairseq2_b200.utils.validation import ValidationError, validate
from fairseq2_b200.utils.yaml import YamlError, dump_yaml, load_yaml


def load_recipe_config(recipe: Recipe, config_files: Sequence[Path] = (), overrides: Mapping[str, Any] | None = None,
                       preset: Any | None = None) -> Any:
    """default dataclass -> unstructure -> merge YAML files (with directives) -> merge overrides -> structure -> validate"""
    base = preset if preset is not None else recipe.config_kls()
    cfg = unstructure(base)
    for f in config_files:
        try:
            docs = load_yaml(Path(f))
        except (YamlError, OSError) as ex:
            raise RecipeConfigParseError(f"The configuration file '{f}' cannot be read: {ex}") from ex
        if len(docs) != 1:
            raise RecipeConfigParseError(f"The configuration file '{f}' must contain exactly one YAML document.")
        doc = process_directives(docs[0], [replace_path_directive(Path(f).resolve().parent), replace_env_directive()])
        cfg = merge_config(cfg, doc)
    if overrides:
        cfg = merge_config(cfg, process_directives(dict(overrides), [replace_env_directive()]))
    try:
        config = structure(cfg, recipe.config_kls)
        validate(config)
    except (StructureError, ValidationError) as ex:
        raise RecipeConfigParseError(f"The recipe configuration is invalid: {ex}") from ex
    return config


def configure_torch(common: CommonSection, rank: int) -> None:
    seed = common.seed
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    t = common.torch
    if t.num_threads is not None:
        torch.set_num_threads(t.num_threads)
    torch.backends.cuda.matmul.allow_tf32 = t.allow_tf32
    torch.backends.cudnn.allow_tf32 = t.allow_tf32
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = t.fp16_reduced_precision
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = t.bf16_reduced_precision
    from fairseq2_b200.models.transformer.sdpa import sdpa_factory_by_name, set_default_sdpa_factory

    set_default_sdpa_factory(sdpa_factory_by_name(t.default_sdpa))


def run_recipe(recipe: Recipe, config: Any, output_dir: Path, *, checkpoint_dir: Path | None = None,
               no_sweep_dir: bool | None = None) -> None:
    common: CommonSection = getattr(config, "common", None) or CommonSection()
    prepare_cluster(common.cluster)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    skip_sweep = common.no_sweep_dir if no_sweep_dir is None else no_sweep_dir
    if not skip_sweep:
        output_dir = output_dir / generate_sweep_tag(unstructure(config), world, common.sweep_format)  # type: ignore[arg-type]
    output_dir.mkdir(parents=True, exist_ok=True)
    configure_logging(debug=common.debug, rank=rank, log_file=output_dir / "logs" / f"rank_{rank}.log")
    if common.debug:
        # per-rank library logs next to the recipe log (fairseq2 ``recipe/internal/logging.py:82-116``)
        os.environ.setdefault("TORCH_DISTRIBUTED_DEBUG", "INFO")
        nccl_dir = output_dir / "logs" / "nccl"
        nccl_dir.mkdir(parents=True, exist_ok=True)
        os.environ.setdefault("NCCL_DEBUG", "INFO")
        os.environ.setdefault("NCCL_DEBUG_FILE", str(nccl_dir / f"rank_{rank}.log"))
        aten_dir = output_dir / "logs" / "aten"
        aten_dir.mkdir(parents=True, exist_ok=True)
        os.environ.setdefault("TORCH_CPP_LOG_LEVEL", "INFO")
    if rank == 0:
        dump_yaml(unstructure(config), output_dir / "config.yaml")
    configure_torch(common, rank)
    log.info("Recipe {} starting; output directory: {}", type(recipe).__name__, output_dir)
    context = RecipeContext(config, output_dir, checkpoint_dir=checkpoint_dir)
    recipe.register(context)
    task = recipe.create_task(context)
    install_stop_signal_handler(task)
    try:
        task.run()
    except TaskStopException:
        log.info("Task stopped at step {} on request.", task.step_nr)
    finally:
        task.close()
        if context._gangs is not None:
            context._gangs.close()
