"""Generation: KV-cache decoding equals full re-computation, samplers, beam
search and step processors."""
from __future__ import annotations

import torch

from fairseq2_b200.generation import (BannedSequenceProcessor, BeamSearchSequenceGenerator,
                                      NGramRepeatBlockProcessor, SamplingSequenceGenerator, TopKSampler, TopPSampler)
from fairseq2_b200.models.llama import create_llama_model, get_llama_config
from fairseq2_b200.nn import BatchLayout, IncrementalStateBag
from fairseq2_b200.ops.sampling import ngram_repeat_block_reference


def _model():
    cfg = get_llama_config("tiny")
    cfg.num_layers = 2
    cfg.vocab_size = 64
    torch.manual_seed(1)
    return create_llama_model(cfg).eval()


def test_incremental_decoding_matches_full_forward() -> None:
    m = _model()
    x = torch.randint(0, 64, (2, 12))
    full = m(x, BatchLayout.of(x))
    bag = IncrementalStateBag(32)
    outs = []
    first = x[:, :5]
    outs.append(m(first, BatchLayout.of(first), state_bag=bag))
    bag.increment_step_nr(5)
    for t in range(5, 12):
        cur = x[:, t:t + 1]
        outs.append(m(cur, BatchLayout.of(cur), state_bag=bag))
        bag.increment_step_nr(1)
    inc = torch.cat(outs, dim=1)
    assert torch.allclose(inc, full, atol=1e-4, rtol=1e-4)


def test_greedy_sampling_is_argmax_continuation() -> None:
    m = _model()
    prompt = torch.randint(1, 64, (2, 4))
    gen = SamplingSequenceGenerator(m, eos_idx=0, sampler=TopKSampler(1), max_gen_len=6, echo_prompt=True)
    out = gen(prompt, BatchLayout.of(prompt))
    for i, hyps in enumerate(out.hypotheses):
        seq = hyps[0].seq
        assert torch.equal(seq[:4], prompt[i])
        # re-derive greedily without a cache
        cur = prompt[i:i + 1]
        for _ in range(seq.numel() - 4):
            nxt = m(cur, BatchLayout.of(cur))[:, -1].argmax(-1, keepdim=True)
            cur = torch.cat([cur, nxt], dim=1)
        assert torch.equal(cur[0, : seq.numel()], seq) or seq[-1] == 0


def test_ragged_prompts_and_num_gens() -> None:
    m = _model()
    prompt = torch.randint(1, 64, (2, 6))
    layout = BatchLayout((2, 6), [3, 6])
    gen = SamplingSequenceGenerator(m, eos_idx=0, sampler=TopPSampler(0.9), num_gens=2, max_gen_len=5,
                                    echo_prompt=True, compute_scores=True)
    out = gen(prompt, layout)
    assert [len(h) for h in out.hypotheses] == [2, 2]
    assert torch.equal(out.hypotheses[0][0].seq[:3], prompt[0, :3])
    assert torch.equal(out.hypotheses[1][0].seq[:6], prompt[1])
    assert out.hypotheses[0][0].seq.numel() <= 3 + 5


def test_beam_search_finds_at_least_greedy_score() -> None:
    m = _model()
    prompt = torch.randint(1, 64, (1, 4))
    beam = BeamSearchSequenceGenerator(m, eos_idx=0, beam_size=3, max_gen_len=5, normalize_scores=False)
    out = beam(prompt, BatchLayout.of(prompt))
    assert 1 <= len(out.hypotheses[0]) <= 3
    scores = [float(h.score) for h in out.hypotheses[0]]
    assert scores == sorted(scores, reverse=True)


def test_step_processors() -> None:
    seqs = torch.tensor([[1, 2, 3, 1, 2], [4, 5, 6, 7, 8]])
    probs = torch.full((2, 10), 0.1)
    NGramRepeatBlockProcessor(3)(seqs, probs)
    assert probs[0, 3] == 0.0 and abs(float(probs[0].sum()) - 0.9) < 1e-6 and abs(float(probs[1].sum()) - 1.0) < 1e-6
    probs = torch.full((2, 10), 0.1)
    BannedSequenceProcessor([torch.tensor([9]), torch.tensor([7, 8, 2])])(seqs, probs)
    assert probs[0, 9] == 0 and probs[1, 9] == 0 and probs[1, 2] == 0 and probs[0, 2] == 0.1
    lp = torch.zeros((2, 10))
    ngram_repeat_block_reference(seqs, lp, 2, float("-inf"))
    assert lp[0, 3] == float("-inf")
