"""Configuration of the batch text generation recipe (cf. fairseq2 ``recipes/lm/generate/config.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from fairseq2_b200.recipe.config import (CommonSection, DatasetSection, GangSection, GeneratorSection, ModelSection,
                                         SequenceGeneratorSection, TokenizerSection)

from .dataset import LM_GENERATE_DATASET


@dataclass(kw_only=True)
class LMGenerateDatasetSection(DatasetSection):
    batch_size: int = 1
    prefetch: int = 4
    encode_mode: str = "prompt"


@dataclass(kw_only=True)
class LMGenerateConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(name="llama3_2_1b_instruct", dtype=torch.bfloat16))
    dataset: LMGenerateDatasetSection = field(default_factory=lambda: LMGenerateDatasetSection(
        family=LM_GENERATE_DATASET))
    tokenizer: TokenizerSection = field(default_factory=lambda: TokenizerSection(name="llama3_2_1b_instruct"))
    gang: GangSection = field(default_factory=GangSection)
    generator: GeneratorSection = field(default_factory=GeneratorSection)
    seq_generator: SequenceGeneratorSection = field(default_factory=lambda: SequenceGeneratorSection(
        name="sampling", config={"max_gen_len": 512}))
    common: CommonSection = field(default_factory=CommonSection)
