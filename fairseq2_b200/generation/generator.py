"""Sequence generators (cf. fairseq2 ``generation/generator.py``,
``sampling/generator.py:41-777``, ``beam_search/generator.py:45-801``,
``beam_search/algo.py:90-107``).

Decoder-only generation: chunked prefill, per-token decode with a KV cache
(``IncrementalStateBag``), temperature, step processors, min/max length and EOS
handling, prompts of different lengths (prompt tokens are forced), ``num_gens``
fan-out, and score normalisation by ``len ** len_penalty``. Beam search keeps
``beam_size`` hypotheses per prompt, expands ``2 * beam_size`` candidates per
step and reorders the cache by the surviving beams.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Sequence

import torch
from torch import Tensor

from fairseq2_b200.generation.sampler import Sampler, TopPSampler
from fairseq2_b200.generation.step_processor import StepProcessor
from fairseq2_b200.models.clm import CausalLM
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag


@dataclass
class Hypothesis:
    seq: Tensor
    score: Tensor | None = None
    step_scores: Tensor | None = None


@dataclass
class SequenceGeneratorOutput:
    hypotheses: list[list[Hypothesis]]
    counters: dict[str, float] = field(default_factory=dict)


class SequenceGenerator(ABC):
    def __init__(self, model: CausalLM, eos_idx: int, pad_idx: int | None = None) -> None:
        self.model, self.eos_idx, self.pad_idx = model, eos_idx, pad_idx
        self._step_hooks: dict[int, Any] = {}

    def register_step_hook(self, hook: Any) -> Any:
        """``hook(prompt_indices, seqs, step_scores, prefill)`` runs after every decoding step with the indices of
        the prompts still being generated and their sequences so far. The returned handle is a context manager
        that removes the hook on exit (or via ``remove()``)."""
        key = max(self._step_hooks, default=-1) + 1
        self._step_hooks[key] = hook
        hooks = self._step_hooks

        class _Handle:
            def remove(self) -> None:
                hooks.pop(key, None)

            def __enter__(self) -> "_Handle":
                return self

            def __exit__(self, *exc: object) -> None:
                self.remove()

        return _Handle()

    @abstractmethod
    def __call__(self, prompt_seqs: Tensor, prompt_layout: BatchLayout) -> SequenceGeneratorOutput: ...


def _prefill(model: CausalLM, seqs: Tensor, length: int, bag: IncrementalStateBag, chunk: int) -> Tensor | None:
    """Feeds ``seqs[:, :length]`` through the model in chunks; returns the logits of the last position."""
    logits = None
    pos = 0
    while pos < length:
        end = min(pos + chunk, length)
        part = seqs[:, pos:end]
        logits = model(part, BatchLayout.of(part), state_bag=bag)
        bag.increment_step_nr(end - pos)
        pos = end
    return logits[:, -1] if logits is not None else None


class SamplingSequenceGenerator(SequenceGenerator):
    def __init__(self, model: CausalLM, eos_idx: int, pad_idx: int | None = None, sampler: Sampler | None = None, *,
                 num_gens: int = 1, min_gen_len: int = 1, max_gen_len: int = 128, max_seq_len: int | None = None,
                 echo_prompt: bool = False, compute_scores: bool = False, normalize_scores: bool = True,
                 temperature: float = 1.0, unk_penalty: float = 0.0, len_penalty: float = 1.0,
                 prefill_chunk_size: int | None = 512, decode_capacity_increment: int | None = 16,
                 step_processors: Sequence[StepProcessor] | None = None, unk_idx: int | None = None) -> None:
        super().__init__(model, eos_idx, pad_idx)
        if min_gen_len < 1:
            raise ValueError(f"`min_gen_len` must be greater than or equal to 1, but is {min_gen_len} instead.")
        if max_gen_len < min_gen_len:
            raise ValueError("`max_gen_len` must be greater than or equal to `min_gen_len`.")
        self.sampler = sampler or TopPSampler(0.9)
        self.num_gens, self.min_gen_len, self.max_gen_len = num_gens, min_gen_len, max_gen_len
        self.max_seq_len = max_seq_len or model.max_seq_len
        self.echo_prompt, self.compute_scores, self.normalize_scores = echo_prompt, compute_scores, normalize_scores
        self.temperature, self.unk_penalty, self.len_penalty = temperature, unk_penalty, len_penalty
        self.prefill_chunk_size = prefill_chunk_size or 1 << 30
        self.decode_capacity_increment = decode_capacity_increment
        self.step_processors = list(step_processors or [])
        self.unk_idx = unk_idx

    @torch.inference_mode()
    def __call__(self, prompt_seqs: Tensor, prompt_layout: BatchLayout) -> SequenceGeneratorOutput:
        model = self.model
        was_training = model.training
        model.eval()
        try:
            return self._generate(prompt_seqs, prompt_layout)
        finally:
            model.train(was_training)

    def _generate(self, prompt_seqs: Tensor, prompt_layout: BatchLayout) -> SequenceGeneratorOutput:
        if prompt_layout.packed:
            raise ValueError("`prompt_seqs` must not be a packed batch.")
        model = self.model
        dev = prompt_seqs.device
        n_prompts = prompt_seqs.shape[0]
        plens = torch.tensor(list(prompt_layout.seq_lens), device=dev)
        if self.num_gens > 1:
            prompt_seqs = prompt_seqs.repeat_interleave(self.num_gens, dim=0)
            plens = plens.repeat_interleave(self.num_gens)
        N = prompt_seqs.shape[0]
        min_plen, max_plen = int(plens.min()), int(plens.max())
        if min_plen < 1:
            raise ValueError("Every prompt must have at least one token.")
        total = min(self.max_seq_len, max_plen + self.max_gen_len)
        pad = self.pad_idx if self.pad_idx is not None else self.eos_idx
        seqs = torch.full((N, total), pad, dtype=prompt_seqs.dtype, device=dev)
        seqs[:, :max_plen] = prompt_seqs[:, :max_plen]
        step_scores = torch.zeros((N, total), device=dev) if self.compute_scores else None
        bag = IncrementalStateBag(total + 1, capacity_increment=self.decode_capacity_increment)
        finished = torch.zeros(N, dtype=torch.bool, device=dev)
        end_pos = torch.full((N,), total, device=dev)
        active = torch.arange(N, device=dev)          # rows still in the cache, in cache order

        # prefill with the part shared by all prompts (all but the last shared token)
        if min_plen > 1:
            _prefill(model, seqs, min_plen - 1, bag, self.prefill_chunk_size)
        num_steps = 0
        for pos in range(min_plen - 1, total - 1):
            cur = seqs[active, pos:pos + 1]
            logits = model(cur, BatchLayout.of(cur), state_bag=bag)[:, -1]
            bag.increment_step_nr(1)
            num_steps += 1
            if self.temperature != 1.0:
                logits = logits / self.temperature
            probs = torch.softmax(logits.float(), dim=-1)
            nxt = pos + 1
            gen_len = nxt - plens[active] + 1     # length of the generation if the sampled token is kept
            for proc in self.step_processors:
                proc(seqs[active, :nxt], probs)
            if self.unk_idx is not None and self.unk_penalty != 0.0:
                probs[:, self.unk_idx] *= max(1.0 - self.unk_penalty, 0.0)
            if self.pad_idx is not None:
                probs[:, self.pad_idx] = 0.0
            probs[gen_len < self.min_gen_len, self.eos_idx] = 0.0
            probs = probs / probs.sum(dim=-1, keepdim=True).clamp(min=1e-30)
            tok = self.sampler.sample(probs)
            at_max = (gen_len >= self.max_gen_len) | (nxt == total - 1)
            tok = torch.where(at_max, torch.full_like(tok, self.eos_idx), tok)
            in_prompt = nxt < plens[active]
            tok = torch.where(in_prompt, seqs[active, nxt], tok)
            seqs[active, nxt] = tok
            if step_scores is not None:
                step_scores[active, nxt] = torch.log(probs.gather(1, tok.unsqueeze(1)).squeeze(1).clamp(min=1e-30))
            if self._step_hooks:
                ss = step_scores[active, :nxt + 1] if step_scores is not None else None
                for hook in self._step_hooks.values():
                    hook(active // self.num_gens, seqs[active, :nxt + 1], ss, False)
            done = (tok == self.eos_idx) & ~in_prompt
            if done.any():
                rows = active[done]
                finished[rows] = True
                end_pos[rows] = nxt + 1
                keep = (~done).nonzero(as_tuple=True)[0]
                if keep.numel() == 0:
                    active = active[:0]
                    break
                bag.reorder(keep)
                active = active[keep]
        end_pos = torch.where(finished, end_pos, torch.full_like(end_pos, total))

        hyps: list[list[Hypothesis]] = [[] for _ in range(n_prompts)]
        ends, pl = end_pos.tolist(), plens.tolist()
        for i in range(N):
            start = 0 if self.echo_prompt else pl[i]
            seq = seqs[i, start:ends[i]]
            score = ss = None
            if step_scores is not None:
                ss = step_scores[i, pl[i]:ends[i]]
                score = ss.sum()
                if self.normalize_scores:
                    score = score / max(ends[i] - pl[i], 1) ** self.len_penalty
            hyps[i // self.num_gens].append(Hypothesis(seq, score, ss))
        if self.compute_scores:
            for h in hyps:
                h.sort(key=lambda x: float(x.score), reverse=True)  # type: ignore[arg-type]
        return SequenceGeneratorOutput(hyps, {"num_decode_steps": num_steps, "cache_bytes": bag.size_bytes()})


class BeamSearchAlgorithm(ABC):
    @abstractmethod
    def step(self, beam_size: int, lprobs: Tensor, scores: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        """``lprobs``: ``(B, V)`` of one prompt's beams, ``scores``: ``(B,)`` cumulative.
        Returns (beam indices, token ids, new scores) of the top ``2 * beam_size`` candidates."""


class StandardBeamSearchAlgorithm(BeamSearchAlgorithm):
    def step(self, beam_size: int, lprobs: Tensor, scores: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        from fairseq2_b200.ops.sampling import beam_topk

        V = lprobs.shape[-1]
        n = lprobs.numel()
        k = min(2 * beam_size, n - 1) if n > 1 else 1
        top, idx = beam_topk(lprobs.unsqueeze(0).float(), scores.unsqueeze(0).float(), k)
        top, idx = top[0].to(lprobs.dtype), idx[0]
        return idx // V, idx % V, top


class BeamSearchSequenceGenerator(SequenceGenerator):
    def __init__(self, model: CausalLM, eos_idx: int, pad_idx: int | None = None,
                 algorithm: BeamSearchAlgorithm | None = None, *, beam_size: int = 5, min_gen_len: int = 1,
                 max_gen_len: int = 128, max_seq_len: int | None = None, echo_prompt: bool = False,
                 normalize_scores: bool = True, temperature: float = 1.0, unk_penalty: float = 0.0,
                 len_penalty: float = 1.0, prefill_chunk_size: int | None = 512,
                 decode_capacity_increment: int | None = 16, step_processors: Sequence[StepProcessor] | None = None,
                 unk_idx: int | None = None) -> None:
        super().__init__(model, eos_idx, pad_idx)
        self.algorithm = algorithm or StandardBeamSearchAlgorithm()
        self.beam_size, self.min_gen_len, self.max_gen_len = beam_size, min_gen_len, max_gen_len
        self.max_seq_len = max_seq_len or model.max_seq_len
        self.echo_prompt, self.normalize_scores = echo_prompt, normalize_scores
        self.temperature, self.unk_penalty, self.len_penalty = temperature, unk_penalty, len_penalty
        self.prefill_chunk_size = prefill_chunk_size or 1 << 30
        self.decode_capacity_increment = decode_capacity_increment
        self.step_processors = list(step_processors or [])
        self.unk_idx = unk_idx

    @torch.inference_mode()
    def __call__(self, prompt_seqs: Tensor, prompt_layout: BatchLayout) -> SequenceGeneratorOutput:
        model = self.model
        was_training = model.training
        model.eval()
        try:
            out = [self._search_one(prompt_seqs[i, : prompt_layout.seq_lens[i]]) for i in range(prompt_seqs.shape[0])]
        finally:
            model.train(was_training)
        return SequenceGeneratorOutput(out)

    def _search_one(self, prompt: Tensor) -> list[Hypothesis]:
        """Beam search for a single prompt (prompts are independent; each has its own cache)."""
        dev = prompt.device
        plen = prompt.numel()
        total = min(self.max_seq_len, plen + self.max_gen_len)
        bag = IncrementalStateBag(total + 1, capacity_increment=self.decode_capacity_increment)
        seqs = prompt.unsqueeze(0)                      # (1, plen): beams grow after the first step
        scores = torch.zeros(1, device=dev)
        if plen > 1:
            _prefill(self.model, seqs, plen - 1, bag, self.prefill_chunk_size)
        finished: list[Hypothesis] = []
        for pos in range(plen - 1, total - 1):
            cur = seqs[:, pos:pos + 1]
            logits = self.model(cur, BatchLayout.of(cur), state_bag=bag)[:, -1]
            bag.increment_step_nr(1)
            if self.temperature != 1.0:
                logits = logits / self.temperature
            lprobs = torch.log_softmax(logits.float(), dim=-1)
            gen_len = pos + 2 - plen
            for proc in self.step_processors:
                proc(seqs, lprobs, lprob=True)
            if self.unk_idx is not None and self.unk_penalty != 0.0:
                lprobs[:, self.unk_idx] -= self.unk_penalty
            if self.pad_idx is not None:
                lprobs[:, self.pad_idx] = float("-inf")
            if gen_len < self.min_gen_len:
                lprobs[:, self.eos_idx] = float("-inf")
            if gen_len >= self.max_gen_len or pos + 1 == total - 1:
                eos = lprobs[:, self.eos_idx].clone()
                lprobs.fill_(float("-inf"))
                lprobs[:, self.eos_idx] = eos
            beam_idx, tok, cand_scores = self.algorithm.step(self.beam_size, lprobs, scores)
            new_beams: list[int] = []
            new_toks: list[int] = []
            new_scores: list[Tensor] = []
            for rank, (b, t, sc) in enumerate(zip(beam_idx.tolist(), tok.tolist(), cand_scores)):
                if not torch.isfinite(sc):
                    continue
                if t == self.eos_idx:
                    if rank >= self.beam_size:
                        continue            # EOS candidates count only within the top `beam_size`
                    full = torch.cat([seqs[b], torch.tensor([t], device=dev, dtype=seqs.dtype)])
                    score = sc / (full.numel() - 1) ** self.len_penalty if self.normalize_scores else sc
                    finished.append(Hypothesis(full if self.echo_prompt else full[plen:], score))
                else:
                    new_beams.append(b)
                    new_toks.append(t)
                    new_scores.append(sc)
                if len(new_beams) == self.beam_size:
                    break
            if len(finished) >= self.beam_size or not new_beams:
                break
            order = torch.tensor(new_beams, device=dev)
            bag.reorder(order)
            seqs = torch.cat([seqs[order], torch.tensor(new_toks, device=dev, dtype=seqs.dtype).unsqueeze(1)], dim=1)
            scores = torch.stack(new_scores)
        finished.sort(key=lambda h: float(h.score), reverse=True)  # type: ignore[arg-type]
        return finished[: self.beam_size]
