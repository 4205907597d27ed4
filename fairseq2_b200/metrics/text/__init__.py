"""Text quality metrics with rank-summable sufficient statistics (cf. fairseq2 ``metrics/text/bleu.py:26-115``,
``metrics/text/chrf.py:23-90``, ``metrics/text/wer.py:24-130``).

Every metric keeps a fixed-size vector of counts that is summed across processes, so the corpus-level score
computed after synchronisation equals the score of the concatenated corpora."""
from __future__ import annotations

import math
import re
from collections import Counter
from typing import Any, Sequence

import numpy as np
import torch
from torch import Tensor

from fairseq2_b200.metrics.aggregation import Metric

_PUNCT = re.compile(r"([\{-\~\[-\` -\&\(-\+\:-\@\/])")
_PERIOD_COMMA_1 = re.compile(r"([^0-9])([\.,])")
_PERIOD_COMMA_2 = re.compile(r"([\.,])([^0-9])")
_DASH = re.compile(r"([0-9])(-)")


def tokenize_13a(line: str) -> list[str]:
    """The WMT ``mteval-v13a`` tokenisation (the default of the reference BLEU metric)."""
    line = line.replace("<skipped>", "").replace("-\n", "").replace("\n", " ")
    line = line.replace("&quot;", '"').replace("&amp;", "&").replace("&lt;", "<").replace("&gt;", ">")
    line = f" {line} "
    line = _PUNCT.sub(r" \1 ", line)
    line = _PERIOD_COMMA_1.sub(r"\1 \2 ", line)
    line = _PERIOD_COMMA_2.sub(r" \1 \2", line)
    line = _DASH.sub(r"\1 \2 ", line)
    return line.split()


def _ngrams(tokens: Sequence[Any], n: int) -> Counter:  # type: ignore[type-arg]
    return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


class BleuMetric(Metric):
    """Corpus BLEU-4 with brevity penalty. State: ``[hyp_len, ref_len, match_1..4, total_1..4]``."""

    state_size = 10
    MAX_ORDER = 4

    def update(self, refs: Sequence[str], hyps: Sequence[str] | None = None, **kw: Any) -> None:  # type: ignore[override]
        if hyps is None or len(refs) != len(hyps):
            raise ValueError("`refs` and `hyps` must be sequences of the same length.")
        acc = np.zeros(self.state_size)
        for ref, hyp in zip(refs, hyps):
            r, h = tokenize_13a(ref), tokenize_13a(hyp)
            acc[0] += len(h)
            acc[1] += len(r)
            for n in range(1, self.MAX_ORDER + 1):
                hn, rn = _ngrams(h, n), _ngrams(r, n)
                acc[1 + n] += sum(min(c, rn[g]) for g, c in hn.items())
                acc[1 + self.MAX_ORDER + n] += max(len(h) - n + 1, 0)
        self.state += torch.from_numpy(acc).to(self.state.device)

    def compute_from(self, state: Tensor) -> Tensor:
        s = state.double().cpu().tolist()
        hyp_len, ref_len = s[0], s[1]
        if hyp_len == 0:
            return torch.zeros((), dtype=torch.float64)
        logp = 0.0
        for n in range(1, self.MAX_ORDER + 1):
            match, total = s[1 + n], s[1 + self.MAX_ORDER + n]
            if total == 0 or match == 0:
                return torch.zeros((), dtype=torch.float64)
            logp += math.log(match / total) / self.MAX_ORDER
        bp = 1.0 if hyp_len > ref_len else math.exp(1.0 - ref_len / hyp_len)
        return torch.tensor(100.0 * bp * math.exp(logp), dtype=torch.float64)


class ChrfMetric(Metric):
    """Corpus chrF (character 6-grams, beta = 2). State: ``[match, hyp_total, ref_total]`` per order."""

    CHAR_ORDER = 6
    BETA = 2.0
    state_size = 3 * 6

    @staticmethod
    def _chars(s: str) -> list[str]:
        return list("".join(s.split()))            # whitespace is ignored, as in the standard definition

    def update(self, refs: Sequence[str], hyps: Sequence[str] | None = None, **kw: Any) -> None:  # type: ignore[override]
        if hyps is None or len(refs) != len(hyps):
            raise ValueError("`refs` and `hyps` must be sequences of the same length.")
        acc = np.zeros(self.state_size)
        for ref, hyp in zip(refs, hyps):
            r, h = self._chars(ref), self._chars(hyp)
            for n in range(1, self.CHAR_ORDER + 1):
                hn, rn = _ngrams(h, n), _ngrams(r, n)
                acc[3 * (n - 1)] += sum(min(c, rn[g]) for g, c in hn.items())
                acc[3 * (n - 1) + 1] += sum(hn.values())
                acc[3 * (n - 1) + 2] += sum(rn.values())
        self.state += torch.from_numpy(acc).to(self.state.device)

    def compute_from(self, state: Tensor) -> Tensor:
        s = state.double().cpu().tolist()
        score, orders = 0.0, 0
        b2 = self.BETA ** 2
        for n in range(self.CHAR_ORDER):
            match, ht, rt = s[3 * n], s[3 * n + 1], s[3 * n + 2]
            if ht == 0 or rt == 0:
                continue
            orders += 1
            p, r = match / ht, match / rt
            if p + r > 0:
                score += (1 + b2) * p * r / (b2 * p + r)
        return torch.tensor(100.0 * score / orders if orders else 0.0, dtype=torch.float64)


def edit_distance(a: Sequence[Any], b: Sequence[Any]) -> int:
    """Levenshtein distance with unit costs; one numpy row per element of ``a``."""
    if len(a) < len(b):
        a, b = b, a
    if not b:
        return len(a)
    vocab: dict[Any, int] = {}
    bi = np.array([vocab.setdefault(x, len(vocab)) for x in b])
    prev = np.arange(len(b) + 1)
    for i, x in enumerate(a, 1):
        xi = vocab.get(x, -1)
        sub = prev[:-1] + (bi != xi)
        cur = np.minimum(prev[1:] + 1, sub)          # deletion / substitution
        # insertions propagate left to right: cur[j] = min(cur[j], cur[j-1] + 1) with cur[-1] = i
        cur = np.minimum.accumulate(np.concatenate(([i], cur)) - np.arange(len(b) + 1)) + np.arange(len(b) + 1)
        prev = cur
    return int(prev[-1])


class WerMetric(Metric):
    """Unit (token) and word error rates in percent. State: ``[unit_err, unit_len, word_err, word_len]``."""

    state_size = 4

    def update(self, refs: Sequence[str], hyps: Sequence[str] | None = None, *,  # type: ignore[override]
               ref_seqs: Sequence[Sequence[int]] | None = None, hyp_seqs: Sequence[Sequence[int]] | None = None,
               **kw: Any) -> None:
        if hyps is None or len(refs) != len(hyps):
            raise ValueError("`refs` and `hyps` must be sequences of the same length.")
        acc = np.zeros(4)
        for i, (ref, hyp) in enumerate(zip(refs, hyps)):
            rw, hw = ref.split(), hyp.split()
            acc[2] += edit_distance(rw, hw)
            acc[3] += len(rw)
            if ref_seqs is not None and hyp_seqs is not None:
                ru, hu = list(ref_seqs[i]), list(hyp_seqs[i])
            else:
                ru, hu = list(ref), list(hyp)
            acc[0] += edit_distance(ru, hu)
            acc[1] += len(ru)
        self.state += torch.from_numpy(acc).to(self.state.device)

    def compute_from(self, state: Tensor) -> Tensor:
        s = state.double().cpu()
        uer = 100.0 * s[0] / s[1] if s[1] > 0 else torch.tensor(-1.0, dtype=torch.float64)
        wer = 100.0 * s[2] / s[3] if s[3] > 0 else torch.tensor(-1.0, dtype=torch.float64)
        return torch.stack([torch.as_tensor(uer, dtype=torch.float64), torch.as_tensor(wer, dtype=torch.float64)])
