"""wav2vec 2.0 self-supervised pre-training and its evaluation (cf. fairseq2 ``recipes/wav2vec2/ssl/recipe.py:41-176``,
``ssl/criterion.py``, ``ssl/metrics.py``, ``ssl/eval/recipe.py``)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
from torch import Tensor

from fairseq2_b200.datasets import SequenceBatch
from fairseq2_b200.datasets.family import register_dataset_family
from fairseq2_b200.evaluator import EvalUnit
from fairseq2_b200.validator import StandardValidator
from fairseq2_b200.metrics import MetricBag
from fairseq2_b200.metrics.aggregation import Mean, Sum
from fairseq2_b200.recipe.base import EvalRecipe, RecipeContext, RecipeModel, TrainRecipe
from fairseq2_b200.recipe.config import (CommonSection, EvaluatorSection, GangSection, LRSchedulerSection,
                                         MixedPrecisionSection, ModelSection, OptimizerSection, RegimeSection,
                                         TrainerSection)
from fairseq2_b200.task import Task
from fairseq2_b200.trainer import TrainUnit

from ..common import (WAV2VEC2_SSL_DATASET, ManifestDatasetConfig, ManifestSpeechDataset, SpeechDatasetSection,
                      open_manifest_dataset)


@dataclass(kw_only=True)
class Wav2Vec2SslLossSection:
    diversity_weight: float = 0.1
    features_penalty_weight: float = 10.0


@dataclass(kw_only=True)
class Wav2Vec2SslConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(family="wav2vec2", arch="base"))
    dataset: SpeechDatasetSection = field(default_factory=lambda: SpeechDatasetSection(family=WAV2VEC2_SSL_DATASET))
    gang: GangSection = field(default_factory=GangSection)
    trainer: TrainerSection = field(default_factory=lambda: TrainerSection(
        data_parallelism="ddp", mixed_precision=MixedPrecisionSection(mode="auto", dtype=torch.bfloat16)))
    loss: Wav2Vec2SslLossSection = field(default_factory=Wav2Vec2SslLossSection)
    optimizer: OptimizerSection = field(default_factory=lambda: OptimizerSection(
        name="adamw", config={"lr": 5e-4, "betas": [0.9, 0.98], "eps": 1e-6, "weight_decay": 0.01}))
    lr_scheduler: LRSchedulerSection | None = field(default_factory=lambda: LRSchedulerSection(
        name="polynomial_decay", config={"num_warmup_steps": 32_000}))
    regime: RegimeSection = field(default_factory=lambda: RegimeSection(
        num_steps=400_000, validate_every_n_steps=5_000, checkpoint_every_n_steps=25_000,
        publish_metrics_every_n_steps=200))
    common: CommonSection = field(default_factory=CommonSection)


@dataclass(kw_only=True)
class Wav2Vec2SslEvalConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(name="wav2vec2_base"))
    dataset: SpeechDatasetSection = field(default_factory=lambda: SpeechDatasetSection(
        family=WAV2VEC2_SSL_DATASET, train_split=None))
    gang: GangSection = field(default_factory=GangSection)
    evaluator: EvaluatorSection = field(default_factory=EvaluatorSection)
    loss: Wav2Vec2SslLossSection = field(default_factory=Wav2Vec2SslLossSection)
    common: CommonSection = field(default_factory=CommonSection)


def _ssl_step(model: RecipeModel, batch: SequenceBatch, bag: MetricBag | None, loss_cfg: Wav2Vec2SslLossSection
              ) -> tuple[Tensor, int]:
    seqs, layout = batch.as_input()
    loss, out = model.module(seqs, layout, diversity_weight=loss_cfg.diversity_weight,
                             features_penalty_weight=loss_cfg.features_penalty_weight)
    n = out.num_targets
    if bag is not None:
        ln2 = math.log(2)
        bag.get("loss", Mean).update(loss.aggregate.detach() / n / ln2, weight=n)
        bag.get("contrastive_loss", Mean).update(loss.contrastive.detach() / n / ln2, weight=n)
        bag.get("diversity_loss", Mean).update(loss.diversity.detach() / n / ln2, weight=n)
        bag.get("features_penalty", Mean).update(loss.features_penalty.detach() / n / ln2, weight=n)
        pred = out.logits.detach().argmax(dim=-1)
        bag.get("accuracy", Mean).update((pred == 0).float().mean(), weight=n)
        q = out.quantizer_output
        bag.get("code_perplexity", Mean).update(q.code_perplexity.detach(), weight=n)
        bag.get("prob_perplexity", Mean).update(q.prob_perplexity.detach(), weight=n)
        bag.get("temperature", Mean).update(torch.tensor(float(q.temperature)), weight=n)
        bag.get("num_examples", Sum).update(batch.num_examples)
        bag.get("num_elements", Sum).update(batch.num_elements)
    return loss.aggregate, n


class Wav2Vec2SslTrainUnit(TrainUnit[SequenceBatch]):
    def __init__(self, model: RecipeModel, loss_cfg: Wav2Vec2SslLossSection) -> None:
        self._model, self._cfg = model, loss_cfg

    def process_batch(self, batch: SequenceBatch, metric_bag: Any | None = None) -> tuple[Tensor, int]:
        return _ssl_step(self._model, batch, metric_bag, self._cfg)

    @property
    def model(self) -> Any:
        return self._model.facade


class Wav2Vec2SslEvalUnit(EvalUnit[SequenceBatch]):
    def __init__(self, model: RecipeModel, loss_cfg: Wav2Vec2SslLossSection, name: str | None = None) -> None:
        self._model, self._cfg, self._name = model, loss_cfg, name

    def process_batch(self, batch: SequenceBatch, metric_bag: MetricBag) -> None:
        _ssl_step(self._model, batch, metric_bag, self._cfg)

    @property
    def name(self) -> str | None:
        return self._name

    @property
    def model(self) -> Any:
        return self._model.facade


def _register() -> None:
    register_dataset_family(WAV2VEC2_SSL_DATASET, ManifestSpeechDataset, ManifestDatasetConfig, open_manifest_dataset)


def _valid_splits(section: SpeechDatasetSection) -> list[str]:
    return [s for s in (section.valid_split or "").split(",") if s]


class Wav2Vec2SslRecipe(TrainRecipe):
    @property
    def config_kls(self) -> type:
        return Wav2Vec2SslConfig

    @property
    def has_static_autograd_graph(self) -> bool:
        return False        # LayerDrop changes which parameters take part in a step

    def register(self, context: RecipeContext) -> None:
        _register()

    def create_task(self, context: RecipeContext) -> Task:
        config: Wav2Vec2SslConfig = context.config
        ds = config.dataset
        model = context.bootstrap_model("model", self)
        dataset = context.open_dataset(ManifestSpeechDataset)
        reader = dataset.create_reader(ds.train_split or "train", context.gangs, ds, train=True,
                                       seed=config.common.seed,
                                       num_accumulate=config.trainer.grad_accumulation.num_batches)
        validator = None
        splits = _valid_splits(ds)
        if splits:
            units = [Wav2Vec2SslEvalUnit(model, config.loss, s if len(splits) > 1 else None) for s in splits]
            readers = [dataset.create_reader(s, context.gangs, ds, train=False) for s in splits]
            validator = StandardValidator(units, readers, context.gangs, checkpoint_manager=context.checkpoint_manager, score_metric="loss", lower_better=True,
                                          metric_recorder=context.create_metric_recorder())
        return context.create_trainer(Wav2Vec2SslTrainUnit(model, config.loss), reader, validator)


class Wav2Vec2SslEvalRecipe(EvalRecipe):
    @property
    def config_kls(self) -> type:
        return Wav2Vec2SslEvalConfig

    def register(self, context: RecipeContext) -> None:
        _register()

    def create_task(self, context: RecipeContext) -> Task:
        config: Wav2Vec2SslEvalConfig = context.config
        ds = config.dataset
        model = context.bootstrap_model("model", self, train=False)
        dataset = context.open_dataset(ManifestSpeechDataset)
        splits = _valid_splits(ds)
        units = [Wav2Vec2SslEvalUnit(model, config.loss, s) for s in splits]
        readers = [dataset.create_reader(s, context.gangs, ds, train=False) for s in splits]
        return context.create_evaluator(units, readers)
