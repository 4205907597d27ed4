"""Instruction fine-tuning of a causal LM (cf. fairseq2 ``recipes/lm/sft/recipe.py:45-208``).

The loss is next-token cross entropy over the response tokens only; the model
computes it with its fused final-projection + cross-entropy so the
``(tokens, vocab)`` logits are never materialised."""
from __future__ import annotations

from typing import Any

from torch import Tensor

from fairseq2_b200.datasets import SequenceBatch
from fairseq2_b200.datasets.family import register_dataset_family
from fairseq2_b200.evaluator import EvalUnit
from fairseq2_b200.validator import StandardValidator
from fairseq2_b200.metrics import MetricBag
from fairseq2_b200.metrics.common import update_nll_loss_metric, update_seq_batch_metrics
from fairseq2_b200.recipe.base import RecipeContext, RecipeModel, TrainRecipe
from fairseq2_b200.task import Task
from fairseq2_b200.trainer import TrainUnit

from ..common import check_model_vocabulary
from .config import LMSFTConfig
from .dataset import (LM_SFT_DATASET, Batching, DataReadOptions, LengthBatching, LMSFTDataset, LMSFTDatasetConfig,
                      PackedBatching, StaticBatching, open_lm_sft_dataset)


class LMSFTRecipe(TrainRecipe):
    @property
    def config_kls(self) -> type:
        return LMSFTConfig

    def register(self, context: RecipeContext) -> None:
        register_dataset_family(LM_SFT_DATASET, LMSFTDataset, LMSFTDatasetConfig, open_lm_sft_dataset)

    def create_task(self, context: RecipeContext) -> Task:
        config: LMSFTConfig = context.config
        ds = config.dataset
        tokenizer = context.load_tokenizer()
        model = context.bootstrap_model("model", self)
        check_model_vocabulary(model.config, tokenizer)
        dataset = context.open_dataset(LMSFTDataset)

        def batching(max_tokens: int) -> Batching:
            if ds.batch_size is not None:
                return StaticBatching(ds.batch_size)
            return PackedBatching(max_tokens) if ds.packed else LengthBatching(max_tokens)

        opts = DataReadOptions(
            batching=batching(ds.max_num_tokens), example_shuffle_window=ds.example_shuffle_window,
            batch_shuffle_window=ds.batch_shuffle_window, num_accumulate=config.trainer.grad_accumulation.num_batches,
            prefetch=ds.prefetch, source_encode_mode=ds.source_encode_mode, target_encode_mode=ds.target_encode_mode,
            chat_mode=ds.chat_mode, seed=config.common.seed)
        reader = dataset.create_reader(ds.train_split, tokenizer, context.gangs, ds.min_seq_len, ds.max_seq_len, opts)
        validator = None
        if ds.valid_split is not None:
            vopts = DataReadOptions(
                batching=batching(ds.max_num_valid_tokens or ds.max_num_tokens), example_shuffle_window=1,
                batch_shuffle_window=1, prefetch=ds.prefetch, source_encode_mode=ds.source_encode_mode,
                target_encode_mode=ds.target_encode_mode, chat_mode=ds.chat_mode, sync_batches=True)
            vreader = dataset.create_reader(ds.valid_split, tokenizer, context.gangs, ds.min_seq_len, ds.max_seq_len,
                                            vopts)
            validator = StandardValidator([LMLossEvalUnit(model)], [vreader], context.gangs, checkpoint_manager=context.checkpoint_manager,
                                          score_metric="nll_loss", lower_better=True,
                                          metric_recorder=context.create_metric_recorder())
        return context.create_trainer(LMSFTUnit(model, config.label_smoothing), reader, validator)


def _lm_loss(model: RecipeModel, batch: SequenceBatch, bag: MetricBag | None, label_smoothing: float = 0.0) -> tuple[Tensor, int]:
    inp, tgt = batch.as_auto_regressive()
    seqs, layout = inp.as_input()
    loss = model.module(seqs, layout, targets=tgt.seqs, target_mask=tgt.target_mask, label_smoothing=label_smoothing)
    n = tgt.num_target_elements
    if bag is not None:
        update_nll_loss_metric(bag, loss, n)
        update_seq_batch_metrics(bag, tgt.num_examples, tgt.num_elements, n, tgt.padding)
    return loss, n


class LMSFTUnit(TrainUnit[SequenceBatch]):
    def __init__(self, model: RecipeModel, label_smoothing: float = 0.0) -> None:
        self._model, self._ls = model, label_smoothing

    def process_batch(self, batch: SequenceBatch, metric_bag: Any | None = None) -> tuple[Tensor, int]:
        return _lm_loss(self._model, batch, metric_bag, self._ls)

    @property
    def model(self) -> Any:
        return self._model.facade


class LMLossEvalUnit(EvalUnit[SequenceBatch]):
    def __init__(self, model: RecipeModel) -> None:
        self._model = model

    def process_batch(self, batch: SequenceBatch, metric_bag: MetricBag) -> None:
        _lm_loss(self._model, batch, metric_bag)

    @property
    def model(self) -> Any:
        return self._model.facade
