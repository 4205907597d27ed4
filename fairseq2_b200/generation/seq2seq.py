"""Sequence-to-sequence generators (cf. fairseq2 ``generation/generator.py:109``,
``sampling/generator.py:209``, ``beam_search/generator.py:212``).

An encoder-decoder model is decoded by the SAME step loops as a decoder-only model: a thin view presents the
decoder (with the encoder output cached in the incremental state bag, where it is reordered together with the
key/value caches) as a causal language model to :class:`SamplingSequenceGenerator` /
:class:`BeamSearchSequenceGenerator`. The source is therefore encoded exactly once per call, and candidate
pruning, ``num_gens`` fan-out and beam reordering need no second implementation.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Sequence

import torch
from torch import Tensor

from fairseq2_b200.generation.generator import (BeamSearchAlgorithm, BeamSearchSequenceGenerator,
                                                SamplingSequenceGenerator, SequenceGeneratorOutput)
from fairseq2_b200.generation.sampler import Sampler
from fairseq2_b200.generation.step_processor import StepProcessor
from fairseq2_b200.models.seq2seq import Seq2SeqModel
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag


class _DecoderView:
    """The decoder of ``model`` conditioned on a fixed source batch, with the call signature of a causal LM."""

    def __init__(self, model: Seq2SeqModel) -> None:
        self.model = model
        self.max_seq_len = model.max_target_seq_len
        self._source: Tensor | None = None
        self._layout: BatchLayout | None = None

    def bind(self, source_seqs: Tensor, source_layout: BatchLayout) -> None:
        self._source, self._layout = source_seqs, source_layout

    @property
    def training(self) -> bool:
        return self.model.training

    def eval(self) -> "_DecoderView":
        self.model.eval()
        return self

    def train(self, mode: bool = True) -> "_DecoderView":
        self.model.train(mode)
        return self

    def parameters(self):  # type: ignore[no-untyped-def]
        return self.model.parameters()

    def __call__(self, seqs: Tensor, layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        src, src_layout = self._source, self._layout
        assert src is not None and src_layout is not None
        fan_out = seqs.shape[0] // src.shape[0] if src.shape[0] else 1
        if fan_out > 1 and seqs.shape[0] == fan_out * src.shape[0]:
            # `num_gens` decoder rows per source row; only the first call reads the source (it is cached after)
            src = src.repeat_interleave(fan_out, dim=0)
            lens = [n for n in src_layout.seq_lens for _ in range(fan_out)]
            src_layout = BatchLayout(tuple(src.shape[:2]), lens, device=src.device)
        return self.model(src, src_layout, seqs, layout, state_bag=state_bag)


class Seq2SeqGenerator(ABC):
    """Generates target sequences for a batch of source sequences, each started from a (possibly empty-but-for-a
    -prefix) target prompt."""

    def __init__(self, model: Seq2SeqModel, eos_idx: int, pad_idx: int | None = None) -> None:
        self.model, self.eos_idx, self.pad_idx = model, eos_idx, pad_idx
        self._view = _DecoderView(model)

    @abstractmethod
    def __call__(self, source_seqs: Tensor, source_seqs_layout: BatchLayout, prompt_seqs: Tensor,
                 prompt_seqs_layout: BatchLayout) -> SequenceGeneratorOutput: ...

    @abstractmethod
    def register_step_hook(self, hook: Any) -> Any: ...


def _check(source_seqs: Tensor, source_layout: BatchLayout, prompt_seqs: Tensor, prompt_layout: BatchLayout) -> None:
    if source_layout.packed or prompt_layout.packed:
        raise ValueError("`source_seqs` and `prompt_seqs` must not be packed batches.")
    if source_seqs.shape[0] != prompt_seqs.shape[0]:
        raise ValueError(f"`source_seqs` and `prompt_seqs` must have the same batch size, but have "
                         f"{source_seqs.shape[0]} and {prompt_seqs.shape[0]} instead.")


class SamplingSeq2SeqGenerator(Seq2SeqGenerator):
    def __init__(self, model: Seq2SeqModel, eos_idx: int, pad_idx: int | None = None, sampler: Sampler | None = None,
                 *, num_gens: int = 1, min_gen_len: int = 1, max_gen_len: tuple[int, int] | int = (1, 128),
                 max_seq_len: int | None = None, echo_prompt: bool = False, compute_scores: bool = False,
                 normalize_scores: bool = True, temperature: float = 1.0, unk_penalty: float = 0.0,
                 len_penalty: float = 1.0, prefill_chunk_size: int | None = 512,
                 decode_capacity_increment: int | None = 16, step_processors: Sequence[StepProcessor] | None = None,
                 unk_idx: int | None = None) -> None:
        """``max_gen_len``: an absolute limit, or ``(a, b)`` meaning ``a * source_len + b`` per call."""
        super().__init__(model, eos_idx, pad_idx)
        self.max_gen_len = max_gen_len
        first = max_gen_len if isinstance(max_gen_len, int) else max(max_gen_len[1], min_gen_len)
        self._gen = SamplingSequenceGenerator(
            self._view, eos_idx, pad_idx, sampler, num_gens=num_gens, min_gen_len=min_gen_len, max_gen_len=first,  # type: ignore[arg-type]
            max_seq_len=max_seq_len, echo_prompt=echo_prompt, compute_scores=compute_scores,
            normalize_scores=normalize_scores, temperature=temperature, unk_penalty=unk_penalty,
            len_penalty=len_penalty, prefill_chunk_size=prefill_chunk_size,
            decode_capacity_increment=decode_capacity_increment, step_processors=step_processors, unk_idx=unk_idx)

    def register_step_hook(self, hook: Any) -> Any:
        return self._gen.register_step_hook(hook)

    def __call__(self, source_seqs, source_seqs_layout, prompt_seqs, prompt_seqs_layout):  # type: ignore[override]
        _check(source_seqs, source_seqs_layout, prompt_seqs, prompt_seqs_layout)
        if not isinstance(self.max_gen_len, int):
            a, b = self.max_gen_len
            self._gen.max_gen_len = max(int(a * max(source_seqs_layout.seq_lens) + b), self._gen.min_gen_len)
        self._view.bind(source_seqs, source_seqs_layout)
        try:
            return self._gen(prompt_seqs, prompt_seqs_layout)
        finally:
            self._view.bind(None, None)  # type: ignore[arg-type]


class BeamSearchSeq2SeqGenerator(Seq2SeqGenerator):
    def __init__(self, model: Seq2SeqModel, eos_idx: int, pad_idx: int | None = None,
                 algorithm: BeamSearchAlgorithm | None = None, *, beam_size: int = 5, min_gen_len: int = 1,
                 max_gen_len: tuple[int, int] | int = (1, 128), max_seq_len: int | None = None,
                 echo_prompt: bool = False, normalize_scores: bool = True, temperature: float = 1.0,
                 unk_penalty: float = 0.0, len_penalty: float = 1.0, prefill_chunk_size: int | None = 512,
                 decode_capacity_increment: int | None = 16, step_processors: Sequence[StepProcessor] | None = None,
                 unk_idx: int | None = None) -> None:
        super().__init__(model, eos_idx, pad_idx)
        self.max_gen_len = max_gen_len
        first = max_gen_len if isinstance(max_gen_len, int) else max(max_gen_len[1], min_gen_len)
        self._gen = BeamSearchSequenceGenerator(
            self._view, eos_idx, pad_idx, algorithm, beam_size=beam_size, min_gen_len=min_gen_len, max_gen_len=first,  # type: ignore[arg-type]
            max_seq_len=max_seq_len, echo_prompt=echo_prompt, normalize_scores=normalize_scores,
            temperature=temperature, unk_penalty=unk_penalty, len_penalty=len_penalty,
            prefill_chunk_size=prefill_chunk_size, decode_capacity_increment=decode_capacity_increment,
            step_processors=step_processors, unk_idx=unk_idx)

    def register_step_hook(self, hook: Any) -> Any:
        return self._gen.register_step_hook(hook)

    @torch.inference_mode()
    def __call__(self, source_seqs, source_seqs_layout, prompt_seqs, prompt_seqs_layout):  # type: ignore[override]
        _check(source_seqs, source_seqs_layout, prompt_seqs, prompt_seqs_layout)
        model = self.model
        was_training = model.training
        model.eval()
        out = []
        try:
            for i in range(source_seqs.shape[0]):
                n = source_seqs_layout.seq_lens[i]
                src = source_seqs[i: i + 1, :n]                     # each source has its own cache and beams
                self._view.bind(src, BatchLayout(tuple(src.shape[:2]), [n], device=src.device))
                if not isinstance(self.max_gen_len, int):
                    a, b = self.max_gen_len
                    self._gen.max_gen_len = max(int(a * n + b), self._gen.min_gen_len)
                out.append(self._gen._search_one(prompt_seqs[i, : prompt_seqs_layout.seq_lens[i]]))
        finally:
            self._view.bind(None, None)  # type: ignore[arg-type]
            model.train(was_training)
        return SequenceGeneratorOutput(out)
