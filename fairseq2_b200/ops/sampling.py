"""Generation-step operators: n-gram repeat blocking, top-p / top-k sampling
and beam-search candidate selection. The CUDA kernels live in
``csrc/generation.cu``; the PyTorch formulations below are the CPU path and
the oracles.

``ngram_repeat_block`` is the B200 counterpart of the reference's only CUDA
kernel (``native/src/fairseq2n/generation/ngram_repeat_block.cu:20-100``): one
thread per start position compares the n-gram beginning there with the last
``n - 1`` tokens and bans the token that followed it.
"""
from __future__ import annotations

import torch
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


def ngram_repeat_block_reference(seqs: Tensor, probs: Tensor, n: int, ban_value: float) -> None:
    N, S = seqs.shape
    if S < n:
        return
    if n == 1:
        probs.scatter_(1, seqs, ban_value)
        return
    last = seqs[:, S - (n - 1):]                                   # (N, n-1)
    windows = seqs.unfold(1, n, 1)                                 # (N, S-n+1, n)
    match = (windows[:, :, : n - 1] == last.unsqueeze(1)).all(dim=2)   # (N, S-n+1)
    banned = windows[:, :, n - 1]
    rows, cols = match.nonzero(as_tuple=True)
    if rows.numel():
        probs[rows, banned[rows, cols]] = ban_value


def ngram_repeat_block(seqs: Tensor, probs: Tensor, n: int, ban_value: float) -> None:
    if use_kernels(seqs, probs) and probs.dtype == torch.float32 and probs.is_contiguous():
        require_ext().ngram_repeat_block(seqs.contiguous(), probs, n, ban_value)
        return
    ngram_repeat_block_reference(seqs, probs, n, ban_value)


def top_p_sample_reference(probs: Tensor, p: float, generator: torch.Generator | None = None) -> Tensor:
    """Nucleus sampling: keep the smallest prefix of the sorted distribution whose mass exceeds ``p``."""
    sorted_probs, idx = torch.sort(probs, dim=-1, descending=True)
    cum = torch.cumsum(sorted_probs, dim=-1)
    mask = (cum - sorted_probs) > p
    sorted_probs = sorted_probs.masked_fill(mask, 0.0)
    sorted_probs = sorted_probs / sorted_probs.sum(dim=-1, keepdim=True)
    choice = torch.multinomial(sorted_probs, 1, generator=generator)
    return idx.gather(-1, choice).squeeze(-1)


def top_k_sample_reference(probs: Tensor, k: int, generator: torch.Generator | None = None) -> Tensor:
    k = min(k, probs.shape[-1])
    topk_probs, idx = torch.topk(probs, k, dim=-1, sorted=False)
    topk_probs = topk_probs / topk_probs.sum(dim=-1, keepdim=True)
    choice = torch.multinomial(topk_probs, 1, generator=generator)
    return idx.gather(-1, choice).squeeze(-1)


def sample_top_p_top_k(probs: Tensor, *, p: float = 1.0, k: int = 0, generator: torch.Generator | None = None,
                       uniform: Tensor | None = None) -> Tensor:
    """Samples one token per row of ``probs`` (fp32, rows sum to 1).

    CUDA: a single kernel per call finds the nucleus/top-k threshold by radix
    selection over the probability bit patterns (no full sort), then walks the
    CDF of the kept entries with one uniform random number per row.
    """
    if use_kernels(probs) and probs.dtype == torch.float32 and probs.is_contiguous():
        if uniform is None:
            uniform = torch.rand(probs.shape[0], device=probs.device, generator=generator)
        return require_ext().sample_top_p_top_k(probs, uniform, float(p), int(k))
    if k > 0:
        return top_k_sample_reference(probs, k, generator)
    return top_p_sample_reference(probs, p, generator)


def beam_topk_reference(lprobs: Tensor, beam_scores: Tensor, k: int) -> tuple[Tensor, Tensor]:
    """``lprobs``: ``[N, beams, V]``, ``beam_scores``: ``[N, beams]`` -> top ``k`` of the summed scores over the
    flattened ``beams*V`` candidates, as ``(scores [N, k], flat indices [N, k])``."""
    cand = (lprobs + beam_scores.unsqueeze(-1)).flatten(1)
    return torch.topk(cand, k, dim=-1)


def beam_topk(lprobs: Tensor, beam_scores: Tensor, k: int) -> tuple[Tensor, Tensor]:
    """Adds the running beam scores and selects the best ``k`` continuations in one kernel, without
    materialising the ``[N, beams*V]`` sum."""
    if (use_kernels(lprobs) and lprobs.dtype == torch.float32 and lprobs.is_contiguous() and k <= 32
            and beam_scores.dtype == torch.float32):
        return require_ext().beam_topk(lprobs, beam_scores.contiguous(), k)
    return beam_topk_reference(lprobs, beam_scores, k)
