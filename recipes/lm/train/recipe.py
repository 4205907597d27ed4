"""Causal LM pre-training on packed text (cf. fairseq2 ``recipes/lm/train/recipe.py``): every position of the
packed buffer is a target and the loss is the sum of next-token cross entropies."""
from __future__ import annotations

from typing import Any

from torch import Tensor

from fairseq2_b200.datasets import SequenceBatch
from fairseq2_b200.datasets.family import register_dataset_family
from fairseq2_b200.metrics.common import update_nll_loss_metric, update_seq_batch_metrics
from fairseq2_b200.recipe.base import RecipeContext, RecipeModel, TrainRecipe
from fairseq2_b200.task import Task
from fairseq2_b200.trainer import TrainUnit

from ..common import check_model_vocabulary
from .config import LMTrainConfig
from .dataset import LM_TRAIN_DATASET, LMTrainDataset, LMTrainDatasetConfig, open_lm_train_dataset


class LMTrainRecipe(TrainRecipe):
    @property
    def config_kls(self) -> type:
        return LMTrainConfig

    def register(self, context: RecipeContext) -> None:
        register_dataset_family(LM_TRAIN_DATASET, LMTrainDataset, LMTrainDatasetConfig, open_lm_train_dataset)

    def create_task(self, context: RecipeContext) -> Task:
        config: LMTrainConfig = context.config
        ds = config.dataset
        tokenizer = context.load_tokenizer()
        model = context.bootstrap_model("model", self)
        check_model_vocabulary(model.config, tokenizer)
        dataset = context.open_dataset(LMTrainDataset)
        reader = dataset.create_reader(tokenizer, context.gangs, max_seq_len=ds.max_seq_len,
                                       max_num_tokens=ds.max_num_tokens,
                                       num_accumulate=config.trainer.grad_accumulation.num_batches,
                                       seed=config.common.seed, prefetch=ds.prefetch, sync_ranks=ds.sync_ranks)
        return context.create_trainer(LMTrainUnit(model), reader)


class LMTrainUnit(TrainUnit[SequenceBatch]):
    def __init__(self, model: RecipeModel) -> None:
        self._model = model

    def process_batch(self, batch: SequenceBatch, metric_bag: Any | None = None) -> tuple[Tensor, int]:
        inp, tgt = batch.as_auto_regressive()
        seqs, layout = inp.as_input()
        loss = self._model.module(seqs, layout, targets=tgt.seqs)
        n = tgt.num_target_elements
        if metric_bag is not None:
            update_nll_loss_metric(metric_bag, loss, n)
            update_seq_batch_metrics(metric_bag, tgt.num_examples, tgt.num_elements, n, tgt.padding)
        return loss, n

    @property
    def model(self) -> Any:
        return self._model.facade
