import random

import torch

from fairseq2_b200.metrics.text import BleuMetric, ChrfMetric, WerMetric, edit_distance, tokenize_13a


def _dp(a, b):  # type: ignore[no-untyped-def]
    d = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        nd = [i]
        for j, y in enumerate(b, 1):
            nd.append(min(d[j] + 1, nd[j - 1] + 1, d[j - 1] + (x != y)))
        d = nd
    return d[-1]


def test_edit_distance_matches_dynamic_programme() -> None:
    random.seed(0)
    for _ in range(300):
        a = [random.randint(0, 4) for _ in range(random.randint(0, 14))]
        b = [random.randint(0, 4) for _ in range(random.randint(0, 14))]
        assert edit_distance(a, b) == _dp(a, b)


def test_bleu() -> None:
    m = BleuMetric()
    m.update(["the cat sat on the mat ."], ["the cat sat on the mat ."])
    assert abs(float(m.compute()) - 100.0) < 1e-9
    # hand-counted clipped matches: unigrams 12/14, bigrams 8/12, trigrams 4/10, 4-grams 2/8; equal lengths
    m = BleuMetric()
    m.update(["the cat is on the mat", "there is a cat on the mat today"],
             ["the cat sat on the mat", "there is a cat on a mat today"])
    import math
    expect = 100 * math.exp((math.log(12 / 14) + math.log(8 / 12) + math.log(4 / 10) + math.log(2 / 8)) / 4)
    assert abs(float(m.compute()) - expect) < 1e-6
    assert tokenize_13a("Hello, world! 3.5 apples.") == ["Hello", ",", "world", "!", "3.5", "apples", "."]


def test_metrics_are_additive_over_shards() -> None:
    refs = ["a quick brown fox", "jumps over the lazy dog", "hello there general kenobi"]
    hyps = ["a quick brown box", "jumped over a lazy dog", "hello there general"]
    for kls in (BleuMetric, ChrfMetric, WerMetric):
        whole, s1, s2 = kls(), kls(), kls()
        whole.update(refs, hyps)
        s1.update(refs[:1], hyps[:1])
        s2.update(refs[1:], hyps[1:])
        assert torch.allclose(whole.compute(), whole.compute_from(s1.state + s2.state))


def test_wer() -> None:
    w = WerMetric()
    w.update(["a b c d"], ["a x c"])
    uer, wer = w.compute().tolist()
    assert abs(wer - 50.0) < 1e-9 and abs(uer - 100.0 * 3 / 7) < 1e-9
