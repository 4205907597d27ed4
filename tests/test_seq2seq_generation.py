"""Sequence-to-sequence generation on a tiny NLLB model: greedy decoding through the generator equals the argmax
continuation computed by full (cache-less) forward passes; beam search is at least as good; the text front ends
feed the tokenizer's target prefix and decode the best hypothesis."""
from __future__ import annotations

import pytest
import torch

from fairseq2_b200.generation import (BeamSearchSeq2SeqGenerator, SamplingSeq2SeqGenerator, SequenceToTextConverter,
                                      TextTranslator, TopKSampler)
from fairseq2_b200.models.nllb import create_nllb_model
from fairseq2_b200.models.nllb.config import nllb_tiny
from fairseq2_b200.nn import BatchLayout

EOS, PAD = 3, 0


def _model():
    torch.manual_seed(2)
    return create_nllb_model(nllb_tiny()).eval()


def _greedy_oracle(m, src, src_layout, prefix, max_new):
    """Argmax continuation of each row by re-running the whole decoder on the growing target."""
    out = []
    for i in range(src.shape[0]):
        n = src_layout.seq_lens[i]
        s = src[i:i + 1, :n]
        sl = BatchLayout((1, n), [n])
        tgt = prefix[i:i + 1].clone()
        for _ in range(max_new):
            logits = m(s, sl, tgt, BatchLayout.of(tgt))[:, -1].float()
            logits[:, PAD] = float("-inf")
            tok = int(logits.argmax(-1))
            tgt = torch.cat([tgt, torch.tensor([[tok]])], dim=1)
            if tok == EOS:
                break
        out.append(tgt[0, prefix.shape[1]:])
    return out


def test_greedy_seq2seq_matches_full_recomputation() -> None:
    m = _model()
    src = torch.randint(4, 200, (3, 9))
    src_layout = BatchLayout((3, 9), [9, 6, 4])
    prefix = torch.tensor([[EOS, 10], [EOS, 11], [EOS, 12]])
    gen = SamplingSeq2SeqGenerator(m, EOS, PAD, TopKSampler(1), max_gen_len=8, compute_scores=True)
    out = gen(src, src_layout, prefix, BatchLayout.of(prefix))
    want = _greedy_oracle(m, src, src_layout, prefix, 8)
    for hyps, w in zip(out.hypotheses, want):
        got = hyps[0].seq
        n = min(got.numel(), w.numel(), 7)       # the generator forces EOS at the length limit
        assert n > 0 and torch.equal(got[:n], w[:n])


def test_num_gens_and_relative_max_len() -> None:
    m = _model()
    src = torch.randint(4, 200, (2, 5))
    prefix = torch.tensor([[EOS], [EOS]])
    gen = SamplingSeq2SeqGenerator(m, EOS, PAD, TopKSampler(5), num_gens=3, max_gen_len=(1, 2))
    out = gen(src, BatchLayout.of(src), prefix, BatchLayout.of(prefix))
    assert [len(h) for h in out.hypotheses] == [3, 3]
    assert all(h.seq.numel() <= 5 + 2 for hyps in out.hypotheses for h in hyps)


def test_beam_search_seq2seq_is_at_least_as_good_as_greedy() -> None:
    m = _model()
    src = torch.randint(4, 200, (2, 7))
    src_layout = BatchLayout((2, 7), [7, 5])
    prefix = torch.tensor([[EOS, 10], [EOS, 10]])
    greedy = SamplingSeq2SeqGenerator(m, EOS, PAD, TopKSampler(1), max_gen_len=6, compute_scores=True)
    beam = BeamSearchSeq2SeqGenerator(m, EOS, PAD, beam_size=4, max_gen_len=6)
    g = greedy(src, src_layout, prefix, BatchLayout.of(prefix))
    b = beam(src, src_layout, prefix, BatchLayout.of(prefix))
    for gh, bh in zip(g.hypotheses, b.hypotheses):
        assert len(bh) >= 1
        assert float(bh[0].score) >= float(gh[0].score) - 0.35   # different length normalisation conventions
    with pytest.raises(ValueError):
        beam(src, src_layout, prefix[:1], BatchLayout.of(prefix[:1]))


class _Enc:
    def __init__(self, prefix):
        self.prefix_indices = prefix

    def __call__(self, text: str) -> torch.Tensor:
        return torch.tensor([4 + (ord(c) % 190) for c in text] + [EOS])


class _Tok:
    class vocab_info:
        pad_idx = PAD

    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False):
        assert task == "translation"
        if mode == "target":
            return _Enc(torch.tensor([EOS, 20 if lang == "fra" else 21]))
        return _Enc(None)

    def create_decoder(self, *, skip_special_tokens=False):
        return lambda seq: " ".join(str(int(t)) for t in seq if not (skip_special_tokens and int(t) in (EOS, PAD)))


def test_text_translator_and_converter() -> None:
    m = _model()
    gen = BeamSearchSeq2SeqGenerator(m, EOS, PAD, beam_size=2, max_gen_len=5)
    tr = TextTranslator(gen, _Tok(), source_lang="eng", target_lang="fra", max_source_len=6)
    text, out = tr("hello world")
    assert isinstance(text, str) and len(out.hypotheses) == 1
    texts, out = tr.batch_translate(["a b", "longer sentence"])
    assert len(texts) == 2 and len(out.hypotheses) == 2
    conv = SequenceToTextConverter(gen, _Tok(), "translation", "deu")
    assert conv.target_prefix.tolist() == [EOS, 21]
    t2, _ = conv(torch.randint(4, 200, (5,)))
    assert isinstance(t2, str)
