"""Configuration of the LM pre-training recipe (cf. fairseq2 ``recipes/lm/train/config.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from fairseq2_b200.recipe.config import (CommonSection, DatasetSection, GangSection, LRSchedulerSection,
                                         MixedPrecisionSection, ModelSection, OptimizerSection, RegimeSection,
                                         TokenizerSection, TrainerSection)

from .dataset import LM_TRAIN_DATASET


@dataclass(kw_only=True)
class LMTrainDatasetSection(DatasetSection):
    max_seq_len: int = 8192
    max_num_tokens: int = 8192 * 2
    prefetch: int = 4
    sync_ranks: bool = False
    """Packed batches have a fixed size, so ranks only need syncing at the end of the data."""


@dataclass(kw_only=True)
class LMTrainConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(family="llama", arch="llama3_8b"))
    dataset: LMTrainDatasetSection = field(default_factory=lambda: LMTrainDatasetSection(family=LM_TRAIN_DATASET))
    tokenizer: TokenizerSection = field(default_factory=lambda: TokenizerSection(name="llama3"))
    gang: GangSection = field(default_factory=GangSection)
    trainer: TrainerSection = field(default_factory=lambda: TrainerSection(
        data_parallelism="fsdp", max_grad_norm=1.0,
        mixed_precision=MixedPrecisionSection(mode="static", dtype=torch.bfloat16)))
    optimizer: OptimizerSection = field(default_factory=lambda: OptimizerSection(
        name="adamw", config={"lr": 3e-4, "betas": [0.9, 0.95], "weight_decay": 0.1}))
    lr_scheduler: LRSchedulerSection | None = field(default_factory=lambda: LRSchedulerSection(
        name="cosine_annealing", config={"num_warmup_steps": 2000, "final_lr_scale": 0.01}))
    regime: RegimeSection = field(default_factory=lambda: RegimeSection(
        num_steps=100_000, checkpoint_every_n_steps=1000, keep_last_n_checkpoints=2,
        publish_metrics_every_n_steps=10))
    common: CommonSection = field(default_factory=CommonSection)
