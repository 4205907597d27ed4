"""Token samplers (cf. fairseq2 ``generation/sampling/sampler.py:31-104``)."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch
from torch import Tensor

from fairseq2_b200.ops.sampling import sample_top_p_top_k


class Sampler(ABC):
    @abstractmethod
    def sample(self, probs: Tensor) -> Tensor:
        """``probs``: ``(N, V)`` fp32 probabilities -> ``(N,)`` token ids."""


class TopPSampler(Sampler):
    def __init__(self, p: float = 0.9) -> None:
        self.p = p

    def sample(self, probs: Tensor) -> Tensor:
        return sample_top_p_top_k(probs, p=self.p)


class TopKSampler(Sampler):
    def __init__(self, k: int) -> None:
        self.k = k

    def sample(self, probs: Tensor) -> Tensor:
        return sample_top_p_top_k(probs, k=self.k)
