"""Batch text generation (cf. fairseq2 ``recipes/lm/generate/recipe.py:45-230``): every data-parallel rank
writes ``output/rank_N.txt`` (human readable) and ``output/rank_N.jsonl``."""
from __future__ import annotations

import json
from typing import Any, TextIO

from fairseq2_b200.datasets import DataReadError, SequenceBatch
from fairseq2_b200.datasets.family import register_dataset_family
from fairseq2_b200.generator import GeneratorUnit
from fairseq2_b200.metrics import MetricBag
from fairseq2_b200.metrics.aggregation import Sum
from fairseq2_b200.recipe.base import GenerationRecipe, RecipeContext, RecipeModel
from fairseq2_b200.task import Task

from ..common import check_model_vocabulary
from .config import LMGenerateConfig
from .dataset import LM_GENERATE_DATASET, LMGenerateDataset, LMGenerateDatasetConfig, open_lm_generate_dataset


class LMGenerateRecipe(GenerationRecipe):
    @property
    def config_kls(self) -> type:
        return LMGenerateConfig

    def register(self, context: RecipeContext) -> None:
        register_dataset_family(LM_GENERATE_DATASET, LMGenerateDataset, LMGenerateDatasetConfig,
                                open_lm_generate_dataset)

    def create_task(self, context: RecipeContext) -> Task:
        config: LMGenerateConfig = context.config
        gangs = context.gangs
        tokenizer = context.load_tokenizer()
        model = context.bootstrap_model("model", self, train=False)
        model.module.eval()
        check_model_vocabulary(model.config, tokenizer)
        text_fp = json_fp = None
        if gangs.tp.rank == 0:
            out = context.output_dir / "output"
            out.mkdir(parents=True, exist_ok=True)
            text_fp = open(out / f"rank_{gangs.dp.rank}.txt", "w", encoding="utf-8")
            json_fp = open(out / f"rank_{gangs.dp.rank}.jsonl", "w", encoding="utf-8")
        generator = context.create_seq_generator(model, tokenizer)
        unit = LMGenerateUnit(model, generator, tokenizer, text_fp, json_fp)
        dataset = context.open_dataset(LMGenerateDataset)
        reader = dataset.create_reader(tokenizer, gangs, batch_size=config.dataset.batch_size,
                                       prefetch=config.dataset.prefetch, encode_mode=config.dataset.encode_mode)
        return context.create_generator(unit, reader)


class LMGenerateUnit(GeneratorUnit[SequenceBatch]):
    def __init__(self, model: RecipeModel, generator: Any, tokenizer: Any, text_stream: TextIO | None,
                 json_stream: TextIO | None) -> None:
        self._model, self._generator = model, generator
        self._decode = tokenizer.create_decoder(skip_special_tokens=False)
        self._text, self._json = text_stream, json_stream

    def process_batch(self, batch: SequenceBatch, metric_bag: MetricBag) -> None:
        ex = batch.example
        if not isinstance(ex, dict) or "prompt" not in ex:
            raise DataReadError("`batch.example` must be a mapping with a 'prompt' entry.")
        seqs, layout = batch.as_input()
        output = self._generator(seqs, layout)
        metric_bag.get("num_examples", Sum).update(batch.num_examples)
        metric_bag.get("num_elements", Sum).update(batch.num_elements)
        metric_bag.get("generator_num_elements", Sum).update(
            sum(int(h[0].seq.numel()) for h in output.hypotheses if h))
        if self._text is None and self._json is None:
            return
        for id_, prompt, hyps in zip(ex["id"], ex["prompt"], output.hypotheses):
            if not hyps:
                raise RuntimeError("The sequence generator returned no hypothesis.")
            h = hyps[0]
            response = self._decode(h.seq)
            score = None if h.score is None else float(h.score)
            steps = None if h.step_scores is None else h.step_scores.tolist()
            if self._text is not None:
                w = self._text.write
                w(f"<<<<< ID >>>>>\n{id_}\n\n<<<<< PROMPT >>>>>\n{prompt}\n\n<<<<< RESPONSE >>>>>\n{response}\n\n")
                w("<<<<< TOKEN INDICES >>>>>\n" + ", ".join(str(t) for t in h.seq.tolist()))
                if score is not None:
                    w(f"\n\n<<<<< SCORE >>>>>\n{score:.8f}")
                if steps is not None:
                    w("\n\n<<<<< STEP SCORES >>>>>\n" + ", ".join(f"{s:.8f}" for s in steps))
                w("\n\n\n============================\n\n\n")
            if self._json is not None:
                json.dump({"id": id_, "prompt": prompt, "response": response, "token_indices": h.seq.tolist(),
                           "score": score, "step_scores": steps}, self._json)
                self._json.write("\n")
        for s in (self._text, self._json):
            if s is not None:
                s.flush()

    def finalize(self, metric_bag: MetricBag) -> None:
        for s in (self._text, self._json):
            if s is not None:
                s.flush()

    @property
    def model(self) -> Any:
        return self._model.facade
