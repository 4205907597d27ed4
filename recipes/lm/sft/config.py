"""Configuration of the instruction fine-tuning recipe (cf. fairseq2 ``recipes/lm/sft/config.py:31-142``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from fairseq2_b200.recipe.config import (CommonSection, DatasetSection, GangSection, LRSchedulerSection,
                                         MixedPrecisionSection, ModelSection, OptimizerSection, RegimeSection,
                                         TokenizerSection, TrainerSection)

from .dataset import LM_SFT_DATASET


@dataclass(kw_only=True)
class LMSFTDatasetSection(DatasetSection):
    train_split: str = "train"
    valid_split: str | None = None
    source_encode_mode: str = "prompt"
    target_encode_mode: str = "prompt_response"
    chat_mode: bool = False
    min_seq_len: int = 1
    max_seq_len: int = 8192
    """Longer examples are dropped."""
    max_num_tokens: int = 8192 * 2
    """Tokens per batch (excluding padding)."""
    batch_size: int | None = None
    """If set, ``max_num_tokens`` is ignored and every batch has this many examples."""
    packed: bool = True
    """Pack examples back to back into fixed buffers of ``max_num_tokens`` tokens."""
    max_num_valid_tokens: int | None = None
    example_shuffle_window: int = 10_000
    batch_shuffle_window: int = 0
    prefetch: int = 4


@dataclass(kw_only=True)
class LMSFTConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(name="llama3_2_1b"))
    dataset: LMSFTDatasetSection = field(default_factory=lambda: LMSFTDatasetSection(family=LM_SFT_DATASET))
    tokenizer: TokenizerSection = field(default_factory=lambda: TokenizerSection(name="llama3_2_1b_instruct"))
    gang: GangSection = field(default_factory=GangSection)
    trainer: TrainerSection = field(default_factory=lambda: TrainerSection(
        data_parallelism="fsdp", max_grad_norm=1.0,
        mixed_precision=MixedPrecisionSection(mode="static", dtype=torch.bfloat16)))
    optimizer: OptimizerSection = field(default_factory=lambda: OptimizerSection(
        name="adamw", config={"lr": 3e-4, "betas": [0.9, 0.95], "weight_decay": 0.1}))
    lr_scheduler: LRSchedulerSection | None = field(default_factory=lambda: LRSchedulerSection(
        name="cosine_annealing", config={"final_lr_scale": 0.2}))
    regime: RegimeSection = field(default_factory=lambda: RegimeSection(
        num_steps=48_000, validate_every_n_steps=4000, checkpoint_every_n_steps=1000, keep_last_n_checkpoints=3,
        keep_checkpoint_every_n_steps=4000, publish_metrics_every_n_steps=10, export_hugging_face=True,
        save_model_only="all_but_last"))
    common: CommonSection = field(default_factory=CommonSection)
    label_smoothing: float = 0.0
