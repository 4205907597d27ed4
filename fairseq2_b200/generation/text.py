"""Text front ends of the generators (cf. fairseq2 ``generation/text.py``)."""
from __future__ import annotations

from typing import Any, Sequence

import torch

from fairseq2_b200.generation.generator import SequenceGenerator, SequenceGeneratorOutput
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
