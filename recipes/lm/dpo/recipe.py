"""Direct preference optimization of a causal LM against a frozen reference policy.

fairseq2 advertises preference optimization and ships the reference-model plumbing
(``recipe/config.py:128`` ``ReferenceModelSection``, ``recipe/base.py:128-149``
``bootstrap_reference_model``); this recipe is the training loop on top of it:

    loss = -log sigmoid(beta * [(log pi(y_w|x) - log ref(y_w|x)) - (log pi(y_l|x) - log ref(y_l|x))])
           + nll_scale * NLL(y_w | x)

Data: JSONL lines with ``src``, ``tgt_chosen`` and ``tgt_rejected``. Chosen and rejected continuations of a
batch run through the policy in ONE forward pass (concatenated along the batch dimension).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Final

import torch
from torch import Tensor
from torch.nn import Module
from torch.nn.functional import logsigmoid

from fairseq2_b200.data import Collater, CollateOptionsOverride, read_sequence
from fairseq2_b200.data.text import read_text
from fairseq2_b200.data.tokenizers import Tokenizer
from fairseq2_b200.datasets import DataPipelineReader, SyncMode
from fairseq2_b200.datasets.family import register_dataset_family
from fairseq2_b200.gang import Gangs
from fairseq2_b200.metrics.aggregation import Mean, Sum
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.recipe.base import RecipeContext, RecipeModel, TrainRecipe
from fairseq2_b200.recipe.config import (CommonSection, DatasetSection, GangSection, LRSchedulerSection,
                                         MixedPrecisionSection, ModelSection, OptimizerSection, ReferenceModelSection,
                                         RegimeSection, TokenizerSection, TrainerSection)
from fairseq2_b200.task import Task
from fairseq2_b200.trainer import TrainUnit

LM_PREFERENCE_DATASET: Final = "lm_preference"


@dataclass(kw_only=True)
class PreferenceDatasetConfig:
    path: Path = Path()


@dataclass(kw_only=True)
class PreferenceDatasetSection(DatasetSection):
    max_seq_len: int = 4096
    batch_size: int = 4
    example_shuffle_window: int = 10_000
    prefetch: int = 4


@dataclass(kw_only=True)
class DPOSection:
    beta: float = 0.1
    nll_scale: float = 0.0
    length_normalization: bool = False


@dataclass(kw_only=True)
class LMDPOConfig:
    model: ModelSection = field(default_factory=lambda: ModelSection(name="llama3_2_1b_instruct"))
    reference_model: ReferenceModelSection | None = field(default_factory=lambda: ReferenceModelSection(
        name="llama3_2_1b_instruct"))
    """``None`` trains reference-free (the reference log-ratios are taken as zero)."""
    dataset: PreferenceDatasetSection = field(default_factory=lambda: PreferenceDatasetSection(
        family=LM_PREFERENCE_DATASET))
    tokenizer: TokenizerSection = field(default_factory=lambda: TokenizerSection(name="llama3_2_1b_instruct"))
    gang: GangSection = field(default_factory=GangSection)
    trainer: TrainerSection = field(default_factory=lambda: TrainerSection(
        data_parallelism="fsdp", max_grad_norm=1.0,
        mixed_precision=MixedPrecisionSection(mode="static", dtype=torch.bfloat16)))
    criterion: DPOSection = field(default_factory=DPOSection)
    optimizer: OptimizerSection = field(default_factory=lambda: OptimizerSection(
        name="adamw", config={"lr": 5.5e-6, "betas": [0.9, 0.95], "weight_decay": 0.1}))
    lr_scheduler: LRSchedulerSection | None = field(default_factory=lambda: LRSchedulerSection(
        name="cosine_annealing", config={"final_lr_scale": 0.2}))
    regime: RegimeSection = field(default_factory=lambda: RegimeSection(
        num_steps=5000, checkpoint_every_n_steps=1000, publish_metrics_every_n_steps=10))
    common: CommonSection = field(default_factory=CommonSection)


@dataclass
class PreferenceBatch:
    chosen: Tensor
    chosen_lens: list[int]
    rejected: Tensor
    rejected_lens: list[int]
    prompt_lens: list[int]

    def to(self, device: torch.device, *, non_blocking: bool = False) -> "PreferenceBatch":
        self.chosen = self.chosen.to(device, non_blocking=non_blocking)
        self.rejected = self.rejected.to(device, non_blocking=non_blocking)
        return self

    @property
    def batch_size(self) -> int:
        return len(self.prompt_lens)


class PreferenceDataset:
    def __init__(self, name: str, path: Path) -> None:
        self._name, self._path = name, Path(path)

    def create_reader(self, tokenizer: Tokenizer, gangs: Gangs, section: PreferenceDatasetSection, *, seed: int = 2,
                      num_accumulate: int = 1) -> DataPipelineReader[PreferenceBatch]:
        path = self._path
        files = sorted(f for f in path.glob("**/*.jsonl") if f.is_file()) if path.is_dir() else [path]
        b = read_sequence([str(f) for f in files])
        b.yield_from(lambda f: read_text(f, rtrim=True, skip_empty=True).map(json.loads).and_return())
        if section.example_shuffle_window != 1:
            b.shuffle(section.example_shuffle_window, seed=seed)
        b.shard(gangs.dp.rank, gangs.dp.size, allow_uneven=True)
        src_enc = tokenizer.create_encoder(mode="prompt")
        tgt_enc = tokenizer.create_encoder(mode="prompt_response")
        max_len = section.max_seq_len

        def encode(ex: dict[str, Any]) -> dict[str, Any]:
            s = src_enc(ex["src"])
            return {"chosen": torch.cat([s, tgt_enc(ex["tgt_chosen"])]),
                    "rejected": torch.cat([s, tgt_enc(ex["tgt_rejected"])]), "prompt_len": len(s)}

        b.map(encode)
        b.filter(lambda ex: max(len(ex["chosen"]), len(ex["rejected"])) <= max_len)
        b.bucket(section.batch_size, drop_remainder=False)
        pad = tokenizer.vocab_info.pad_idx
        b.map(Collater(pad_value=pad if pad is not None else 0))
        b.prefetch(section.prefetch)

        def to_batch(ex: dict[str, Any]) -> PreferenceBatch:
            c, r = ex["chosen"], ex["rejected"]
            pl = ex["prompt_len"]
            pl = pl.tolist() if isinstance(pl, Tensor) else list(pl)
            return PreferenceBatch(c["seqs"], list(c["seq_lens"]), r["seqs"], list(r["seq_lens"]), pl)

        b.map(to_batch)
        return DataPipelineReader(self._name, "train", b.and_return(), gangs.dp, num_accumulate=num_accumulate,
                                  drop_remainder=False, sync=True, sync_mode=SyncMode.UNTIL_FIRST)


def sequence_logps(model: Module, seqs: Tensor, lens: list[int], prompt_lens: list[int]) -> tuple[Tensor, Tensor]:
    """Sum of response-token log-probabilities per sequence and the number of response tokens."""
    inp, tgt = seqs[:, :-1], seqs[:, 1:]
    layout = BatchLayout(tuple(inp.shape), [max(l - 1, 1) for l in lens], device=seqs.device)
    logits = model(inp, layout)
    lp = torch.log_softmax(logits.float(), dim=-1).gather(-1, tgt.unsqueeze(-1)).squeeze(-1)
    pos = torch.arange(tgt.shape[1], device=seqs.device).unsqueeze(0)
    lens_t = torch.tensor(lens, device=seqs.device).unsqueeze(1)
    pl_t = torch.tensor(prompt_lens, device=seqs.device).unsqueeze(1)
    mask = (pos >= pl_t - 1) & (pos < lens_t - 1)        # target position t predicts token t + 1
    return (lp * mask).sum(dim=1), mask.sum(dim=1)


class DPOTrainUnit(TrainUnit[PreferenceBatch]):
    def __init__(self, model: RecipeModel, reference: Module | None, cfg: DPOSection) -> None:
        self._model, self._ref, self._cfg = model, reference, cfg

    def _both(self, module: Module, batch: PreferenceBatch) -> tuple[Tensor, Tensor, Tensor, Tensor]:
        n = batch.batch_size
        w = max(batch.chosen.shape[1], batch.rejected.shape[1])
        pad = lambda t: torch.nn.functional.pad(t, (0, w - t.shape[1]))  # noqa: E731
        seqs = torch.cat([pad(batch.chosen), pad(batch.rejected)], dim=0)
        lp, cnt = sequence_logps(module, seqs, batch.chosen_lens + batch.rejected_lens, batch.prompt_lens * 2)
        return lp[:n], lp[n:], cnt[:n], cnt[n:]

    def process_batch(self, batch: PreferenceBatch, metric_bag: Any | None = None) -> tuple[Tensor, int]:
        cfg = self._cfg
        pc, pr, nc, nr = self._both(self._model.module, batch)
        if self._ref is not None:
            with torch.no_grad():
                rc, rr, _, _ = self._both(self._ref, batch)
        else:
            rc, rr = torch.zeros_like(pc), torch.zeros_like(pr)
        if cfg.length_normalization:
            pc_n, pr_n, rc, rr = pc / nc, pr / nr, rc / nc, rr / nr
        else:
            pc_n, pr_n = pc, pr
        margin = cfg.beta * ((pc_n - rc) - (pr_n - rr))
        dpo = -logsigmoid(margin).sum()
        nll = -pc.sum()
        n = batch.batch_size
        # the trainer divides the loss by the returned count: scale the NLL term so that it is per chosen token
        loss = dpo + cfg.nll_scale * nll * n / nc.sum().clamp(min=1)
        if metric_bag is not None:
            metric_bag.get("dpo_loss", Mean).update(dpo.detach() / n, weight=n)
            metric_bag.get("nll_loss", Mean).update(nll.detach() / nc.sum() / math.log(2), weight=int(nc.sum()))
            metric_bag.get("reward_accuracy", Mean).update((margin.detach() > 0).float().mean(), weight=n)
            metric_bag.get("chosen_logps", Mean).update(pc.detach().mean(), weight=n)
            metric_bag.get("rejected_logps", Mean).update(pr.detach().mean(), weight=n)
            metric_bag.get("num_examples", Sum).update(n)
        return loss, n

    @property
    def model(self) -> Any:
        return self._model.facade


class LMDPORecipe(TrainRecipe):
    @property
    def config_kls(self) -> type:
        return LMDPOConfig

    def register(self, context: RecipeContext) -> None:
        register_dataset_family(LM_PREFERENCE_DATASET, PreferenceDataset, PreferenceDatasetConfig,
                                lambda name, cfg: PreferenceDataset(name, cfg.path))

    def create_task(self, context: RecipeContext) -> Task:
        config: LMDPOConfig = context.config
        tokenizer = context.load_tokenizer()
        model = context.bootstrap_model("model", self)
        reference = context.bootstrap_reference_model("reference_model", self) \
            if config.reference_model is not None else None
        dataset = context.open_dataset(PreferenceDataset)
        reader = dataset.create_reader(tokenizer, context.gangs, config.dataset, seed=config.common.seed,
                                       num_accumulate=config.trainer.grad_accumulation.num_batches)
        return context.create_trainer(DPOTrainUnit(model, reference, config.criterion), reader)
