"""wav2vec 2.0 CTC fine-tuning and evaluation (cf. fairseq2 ``recipes/wav2vec2/asr/recipe.py:52-282``,
``asr/criterion.py``, ``asr/wer_calculator.py``, ``asr/eval/recipe.py``): the encoder can be initialised from a
pre-trained SSL model and kept frozen for the first steps; validation reports unit and word error rates from
greedy CTC decoding."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, TextIO

import torch
from torch import Tensor
from torch.nn import Module

from fairseq2_b200.datasets import Seq2SeqBatch
from fairseq2_b200.datasets.family import register_dataset_family
from fairseq2_b200.evaluator import EvalUnit
from fairseq2_b200.validator import StandardValidator
from fairseq2_b200.logging import log
from fairseq2_b200.metrics import MetricBag
from fairseq2_b200.metrics.aggregation import Mean, Sum
from fairseq2_b200.metrics.text import WerMetric
from fairseq2_b200.recipe.base import EvalRecipe, RecipeContext, RecipeModel, TrainRecipe
from fairseq2_b200.recipe.config import (CommonSection, EvaluatorSection, GangSection, LRSchedulerSection,
                                         MixedPrecisionSection, ModelSection, OptimizerSection, ReferenceModelSection,
                                         RegimeSection, TokenizerSection, TrainerSection)
from fairseq2_b200.task import Task
from fairseq2_b200.trainer import TrainUnit

from ..common import (WAV2VEC2_ASR_DATASET, ManifestDatasetConfig, ManifestSpeechDataset, SpeechDatasetSection,
                      open_manifest_dataset)


@dataclass(kw_only=True)
class Wav2Vec2AsrTrainerSection(TrainerSection):
    freeze_encoder_for_n_steps: int = 10_000
    """The encoder is frozen for this many steps while the output projection warms up."""


@dataclass(kw_only=True)
class Wav2Vec2AsrConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(family="wav2vec2_asr", arch="base_10h"))
    pretrained_model: ReferenceModelSection | None = None
    """An SSL wav2vec 2.0 model whose front end and encoder initialise the ASR model."""
    dataset: SpeechDatasetSection = field(default_factory=lambda: SpeechDatasetSection(
        family=WAV2VEC2_ASR_DATASET, min_audio_len=1, max_audio_len=640_000, max_num_elements=3_200_000,
        normalize_audio=False, no_padding=False))
    tokenizer: TokenizerSection = field(default_factory=lambda: TokenizerSection(name="librispeech_asr"))
    gang: GangSection = field(default_factory=GangSection)
    trainer: Wav2Vec2AsrTrainerSection = field(default_factory=lambda: Wav2Vec2AsrTrainerSection(
        data_parallelism="ddp", mixed_precision=MixedPrecisionSection(mode="auto", dtype=torch.bfloat16)))
    optimizer: OptimizerSection = field(default_factory=lambda: OptimizerSection(
        name="adamw", config={"lr": 5e-5, "betas": [0.9, 0.98]}))
    lr_scheduler: LRSchedulerSection | None = field(default_factory=lambda: LRSchedulerSection(
        name="tri_stage", config={"stage_ratio": [0.1, 0.4, 0.5], "start_lr_scale": 0.01, "final_lr_scale": 0.05}))
    regime: RegimeSection = field(default_factory=lambda: RegimeSection(
        num_steps=20_000, validate_after_n_steps=10_000, validate_every_n_steps=1_000,
        checkpoint_every_n_steps=5_000, publish_metrics_every_n_steps=200))
    common: CommonSection = field(default_factory=CommonSection)


@dataclass(kw_only=True)
class Wav2Vec2AsrEvalConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(name="wav2vec2_asr_base_10h"))
    dataset: SpeechDatasetSection = field(default_factory=lambda: SpeechDatasetSection(
        family=WAV2VEC2_ASR_DATASET, train_split=None, valid_split="test_other", min_audio_len=1,
        max_audio_len=640_000, max_num_elements=3_200_000, no_padding=False))
    tokenizer: TokenizerSection = field(default_factory=lambda: TokenizerSection(name="librispeech_asr"))
    gang: GangSection = field(default_factory=GangSection)
    evaluator: EvaluatorSection = field(default_factory=EvaluatorSection)
    common: CommonSection = field(default_factory=CommonSection)


def ctc_greedy_decode(logits: Tensor, lens: list[int], blank: int = 0) -> list[list[int]]:
    """Arg-max path with repeats collapsed and blanks removed."""
    best = logits.argmax(dim=-1).cpu()
    out = []
    for row, n in zip(best, lens):
        r = row[:n]
        keep = torch.ones(n, dtype=torch.bool)
        keep[1:] = r[1:] != r[:-1]
        r = r[keep]
        out.append(r[r != blank].tolist())
    return out


class Wav2Vec2AsrTrainUnit(TrainUnit[Seq2SeqBatch]):
    def __init__(self, model: RecipeModel, freeze_encoder_for_n_steps: int) -> None:
        self._model, self._freeze_n = model, freeze_encoder_for_n_steps
        self._frozen: bool | None = None

    def set_step_nr(self, step_nr: int) -> None:
        base: Module = self._model.base_module
        frozen = step_nr <= self._freeze_n
        if frozen == self._frozen:
            return
        if self._frozen is not None or frozen:
            log.info("{} the encoder at step {}.", "Freezing" if frozen else "Unfreezing", step_nr)
        for part in (base.encoder_frontend, base.encoder):
            part.requires_grad_(not frozen)
        masker = getattr(base, "masker", None)
        if masker is not None:
            masker.requires_grad_(not frozen)
        self._frozen = frozen

    def process_batch(self, batch: Seq2SeqBatch, metric_bag: Any | None = None) -> tuple[Tensor, int]:
        seqs, layout = batch.as_source_input()
        tgt, tgt_layout = batch.as_target_input()
        loss = self._model.module(seqs, layout, tgt, tgt_layout)
        n = batch.batch_size
        if metric_bag is not None:
            metric_bag.get("ctc_loss", Mean).update(loss.detach() / n / math.log(2), weight=n)
            metric_bag.get("num_examples", Sum).update(batch.num_examples)
            metric_bag.get("num_source_elements", Sum).update(batch.num_source_elements)
            metric_bag.get("num_target_elements", Sum).update(batch.num_target_elements)
        return loss, n

    @property
    def model(self) -> Any:
        return self._model.facade


class Wav2Vec2AsrEvalUnit(EvalUnit[Seq2SeqBatch]):
    def __init__(self, model: RecipeModel, tokenizer: Any, name: str | None = None,
                 ref_stream: TextIO | None = None, hyp_stream: TextIO | None = None) -> None:
        self._model, self._name = model, name
        self._decode = tokenizer.create_decoder(skip_special_tokens=True)
        self._pad, self._blank = tokenizer.vocab_info.pad_idx, 0
        self._ref, self._hyp = ref_stream, hyp_stream

    def process_batch(self, batch: Seq2SeqBatch, metric_bag: MetricBag) -> None:
        seqs, layout = batch.as_source_input()
        tgt, tgt_layout = batch.as_target_input()
        loss, logits, logits_layout = self._model.module(seqs, layout, tgt, tgt_layout, return_logits=True)
        n = batch.batch_size
        metric_bag.get("ctc_loss", Mean).update(loss.detach() / n / math.log(2), weight=n)
        hyp_ids = ctc_greedy_decode(logits, list(logits_layout.seq_lens), self._blank)
        ref_ids = [row[:m].tolist() for row, m in zip(tgt.cpu(), tgt_layout.seq_lens)]
        refs = [self._decode(torch.tensor(r)) for r in ref_ids]
        hyps = [self._decode(torch.tensor(h)) for h in hyp_ids]
        wer = metric_bag.get("wer", WerMetric)
        wer.update(refs, hyps, ref_seqs=ref_ids, hyp_seqs=hyp_ids)
        if self._ref is not None and self._hyp is not None:
            for r, h in zip(refs, hyps):
                self._ref.write(r + "\n")
                self._hyp.write(h + "\n")

    def process_metric_values(self, values: dict[str, Any]) -> None:
        pair = values.pop("wer", None)
        if pair is not None:
            values["uer"], values["wer"] = float(pair[0]), float(pair[1])

    @property
    def name(self) -> str | None:
        return self._name

    @property
    def model(self) -> Any:
        return self._model.facade


def _register() -> None:
    register_dataset_family(WAV2VEC2_ASR_DATASET, ManifestSpeechDataset, ManifestDatasetConfig, open_manifest_dataset)


class Wav2Vec2AsrRecipe(TrainRecipe):
    @property
    def config_kls(self) -> type:
        return Wav2Vec2AsrConfig

    @property
    def has_static_autograd_graph(self) -> bool:
        return False

    def register(self, context: RecipeContext) -> None:
        _register()

    def setup_model(self, context: RecipeContext, model: Module, newly_initialized: bool) -> Module:
        config: Wav2Vec2AsrConfig = context.config
        if config.pretrained_model is not None and newly_initialized:
            pt = context.bootstrap_reference_model("pretrained_model")
            log.info("Initialising the encoder from the pre-trained model.")
            model.encoder_frontend.load_state_dict(pt.encoder_frontend.state_dict())
            model.encoder.load_state_dict(pt.encoder.state_dict())
            if getattr(model, "masker", None) is not None and getattr(pt, "masker", None) is not None:
                model.masker.load_state_dict(pt.masker.state_dict())
        # the convolutional feature extractor is never fine-tuned
        fe = getattr(model.encoder_frontend, "feature_extractor", None)
        if fe is not None:
            fe.requires_grad_(False)
        return model

    def create_task(self, context: RecipeContext) -> Task:
        config: Wav2Vec2AsrConfig = context.config
        ds = config.dataset
        tokenizer = context.load_tokenizer()
        model = context.bootstrap_model("model", self)
        dataset = context.open_dataset(ManifestSpeechDataset)
        reader = dataset.create_reader(ds.train_split or "train", context.gangs, ds, tokenizer=tokenizer, train=True,
                                       seed=config.common.seed,
                                       num_accumulate=config.trainer.grad_accumulation.num_batches)
        validator = None
        splits = [s for s in (ds.valid_split or "").split(",") if s]
        if splits:
            units = [Wav2Vec2AsrEvalUnit(model, tokenizer, s if len(splits) > 1 else None) for s in splits]
            readers = [dataset.create_reader(s, context.gangs, ds, tokenizer=tokenizer, train=False) for s in splits]
            validator = StandardValidator(units, readers, context.gangs, checkpoint_manager=context.checkpoint_manager, score_metric="wer", lower_better=True,
                                          metric_recorder=context.create_metric_recorder())
        unit = Wav2Vec2AsrTrainUnit(model, config.trainer.freeze_encoder_for_n_steps)
        return context.create_trainer(unit, reader, validator)


class Wav2Vec2AsrEvalRecipe(EvalRecipe):
    @property
    def config_kls(self) -> type:
        return Wav2Vec2AsrEvalConfig

    def register(self, context: RecipeContext) -> None:
        _register()

    def create_task(self, context: RecipeContext) -> Task:
        config: Wav2Vec2AsrEvalConfig = context.config
        ds = config.dataset
        tokenizer = context.load_tokenizer()
        model = context.bootstrap_model("model", self, train=False)
        dataset = context.open_dataset(ManifestSpeechDataset)
        splits = [s for s in (ds.valid_split or "").split(",") if s]
        out = context.output_dir / "transcriptions"
        out.mkdir(parents=True, exist_ok=True)
        rank = context.gangs.dp.rank
        units, readers = [], []
        for s in splits:
            ref = open(out / f"{s}_rank_{rank}.ref.txt", "w", encoding="utf-8")
            hyp = open(out / f"{s}_rank_{rank}.hyp.txt", "w", encoding="utf-8")
            units.append(Wav2Vec2AsrEvalUnit(model, tokenizer, s, ref, hyp))
            readers.append(dataset.create_reader(s, context.gangs, ds, tokenizer=tokenizer, train=False))
        return context.create_evaluator(units, readers)
