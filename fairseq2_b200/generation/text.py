"""Text front ends of the generators (cf. fairseq2 ``generation/text.py``)."""
from __future__ import annotations

from typing import Any, Sequence

import torch

from torch import Tensor

from fairseq2_b200.generation.generator import SequenceGenerator, SequenceGeneratorOutput
from fairseq2_b200.generation.seq2seq import Seq2SeqGenerator
from fairseq2_b200.nn.batch_layout import BatchLayout


class TextCompleter:
    """Encodes prompts, runs a sequence generator and decodes the best hypothesis."""

    def __init__(self, generator: SequenceGenerator, tokenizer: Any) -> None:
        self.generator = generator
        self.encoder = tokenizer.create_encoder(mode="prompt")
        self.decoder = tokenizer.create_decoder(skip_special_tokens=True)

    def __call__(self, prompt: str) -> tuple[str, SequenceGeneratorOutput]:
        texts, out = self.batch_complete([prompt])
        return texts[0], out

    def batch_complete(self, prompts: Sequence[str]) -> tuple[list[str], SequenceGeneratorOutput]:
        device = next(self.generator.model.parameters()).device
        enc = [self.encoder(p).to(device) for p in prompts]
        lens = [e.numel() for e in enc]
        width = max(lens)
        pad = self.generator.pad_idx if self.generator.pad_idx is not None else self.generator.eos_idx
        seqs = torch.full((len(enc), width), pad, dtype=enc[0].dtype, device=device)
        for i, e in enumerate(enc):
            seqs[i, : e.numel()] = e
        out = self.generator(seqs, BatchLayout((len(enc), width), lens, device=device))
        texts = [self.decoder(h[0].seq) if h else "" for h in out.hypotheses]
        return texts, out


class SequenceToTextConverter:
    """Runs a sequence-to-sequence generator on source sequences (token ids or feature frames) and decodes the best
    hypothesis to text; the target prompt is the prefix that the tokenizer prescribes for ``task`` and
    ``target_lang`` (cf. fairseq2 ``generation/text.py:27-159``)."""

    def __init__(self, generator: Seq2SeqGenerator, tokenizer: Any, task: str, target_lang: str | None = None, *,
                 skip_special_tokens: bool = False) -> None:
        self.generator = generator
        device = next(generator.model.parameters()).device
        enc = tokenizer.create_encoder(task=task, lang=target_lang, mode="target", device=device)
        prefix = enc.prefix_indices
        if prefix is None:
            raise ValueError("`tokenizer` must specify a prefix sequence for the target language.")
        self.target_prefix = prefix.to(device)
        self.decoder = tokenizer.create_decoder(skip_special_tokens=skip_special_tokens)

    def __call__(self, source_seq: Tensor) -> tuple[str, SequenceGeneratorOutput]:
        src = source_seq.unsqueeze(0)
        texts, out = self.batch_convert(src, BatchLayout(tuple(src.shape[:2]), [src.shape[1]], device=src.device))
        return texts[0], out

    def batch_convert(self, source_seqs: Tensor, source_seqs_layout: BatchLayout
                      ) -> tuple[list[str], SequenceGeneratorOutput]:
        if len(source_seqs) == 0:
            raise ValueError("`source_seqs` must contain at least one element, but is empty instead.")
        n = source_seqs.shape[0]
        prompts = self.target_prefix.unsqueeze(0).expand(n, -1).contiguous()
        layout = BatchLayout(tuple(prompts.shape[:2]), [prompts.shape[1]] * n, device=prompts.device)
        out = self.generator(source_seqs, source_seqs_layout, prompts, layout)
        texts = []
        for i, hyps in enumerate(out.hypotheses):
            if not hyps:
                raise RuntimeError(f"The sequence generator returned no hypothesis at index {i}.")
            texts.append(self.decoder(hyps[0].seq))
        return texts, out


class TextTranslator:
    """Text in ``source_lang`` to text in ``target_lang`` (cf. fairseq2 ``generation/text.py:162-260``)."""

    def __init__(self, generator: Seq2SeqGenerator, tokenizer: Any, source_lang: str | None = None,
                 target_lang: str | None = None, *, max_source_len: int | None = None) -> None:
        if max_source_len is not None and max_source_len <= 0:
            raise ValueError(f"`max_source_len` must be greater than or equal to 1, but is {max_source_len} instead.")
        self.converter = SequenceToTextConverter(generator, tokenizer, "translation", target_lang,
                                                 skip_special_tokens=True)
        pad_idx = tokenizer.vocab_info.pad_idx
        if pad_idx is None:
            raise ValueError("`vocab_info` of `tokenizer` must have a PAD symbol defined.")
        self.pad_idx = pad_idx
        self.device = next(generator.model.parameters()).device
        self.source_encoder = tokenizer.create_encoder(task="translation", lang=source_lang, mode="source",
                                                       device=self.device)
        self.max_source_len = max_source_len

    def __call__(self, source_text: str) -> tuple[str, SequenceGeneratorOutput]:
        seq = self.source_encoder(source_text).to(self.device)
        if self.max_source_len:
            seq = seq[: self.max_source_len]
        return self.converter(seq)

    def batch_translate(self, source_texts: Sequence[str]) -> tuple[list[str], SequenceGeneratorOutput]:
        if len(source_texts) == 0:
            raise ValueError("`source_texts` must contain at least one element, but is empty instead.")
        seqs = [self.source_encoder(t).to(self.device) for t in source_texts]
        if self.max_source_len:
            seqs = [s[: self.max_source_len] for s in seqs]
        lens = [s.numel() for s in seqs]
        batch = torch.full((len(seqs), max(lens)), self.pad_idx, dtype=seqs[0].dtype, device=self.device)
        for i, s in enumerate(seqs):
            batch[i, : s.numel()] = s
        return self.converter.batch_convert(batch, BatchLayout(tuple(batch.shape), lens, device=self.device))
