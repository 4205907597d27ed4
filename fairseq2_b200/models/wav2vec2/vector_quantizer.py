"""Gumbel-softmax product quantizer (cf. fairseq2 ``models/wav2vec2/vector_quantizer.py:26-218``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.typing import DataType, Device


@dataclass
class VectorQuantizerOutput:
    quantized_vectors: Tensor
    cb: Tensor | None
    num_codebooks: int
    num_codebook_entries: int
    code_perplexity: Tensor
    prob_perplexity: Tensor
    temperature: float

    def compute_loss(self) -> Tensor:
        n = self.num_codebooks * self.num_codebook_entries
        return (n - self.prob_perplexity) / n

    def get_target_indices(self, num_codebooks: int) -> Tensor:
        if self.cb is None:
            raise ValueError("The codebook indices were not recorded.")
        return self.cb.argmax(dim=-1).view(-1, num_codebooks)[..., :num_codebooks].detach()


class VectorQuantizer(Module, ABC):
    def __init__(self, input_dim: int, output_dim: int) -> None:
        super().__init__()
        self.input_dim, self.output_dim = input_dim, output_dim

    @abstractmethod
    def forward(self, x: Tensor) -> VectorQuantizerOutput: ...


class GumbelVectorQuantizer(VectorQuantizer):
    """``G`` codebooks of ``V`` entries of size ``output_dim / G``; during training entries are drawn with the
    straight-through Gumbel softmax at an exponentially decayed temperature, at inference by arg-max."""

    def __init__(self, input_dim: int, output_dim: int, num_codebooks: int, num_codebook_entries: int, *,
                 codebook_sampling_temperature: tuple[float, float, float], device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(input_dim, output_dim)
        if output_dim % num_codebooks:
            raise ValueError(f"`output_dim` ({output_dim}) must be a multiple of `num_codebooks` ({num_codebooks}).")
        self.num_codebooks, self.num_codebook_entries = num_codebooks, num_codebook_entries
        self.max_temp, self.min_temp, self.temp_decay = codebook_sampling_temperature
        if self.max_temp < self.min_temp:
            raise ValueError("The maximum sampling temperature must be greater than or equal to the minimum.")
        entry_dim = output_dim // num_codebooks
        self.entries = Parameter(torch.empty((1, num_codebooks * num_codebook_entries, entry_dim), device=device,
                                             dtype=dtype))
        self.entry_proj = Linear(input_dim, num_codebooks * num_codebook_entries, bias=True,
                                 init_fn=_init_entry_projection, device=device, dtype=dtype)
        self.register_buffer("num_updates", torch.zeros((), device=device, dtype=torch.int64))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.entries.device.type != "meta":
            torch.nn.init.uniform_(self.entries)
            self.num_updates.zero_()

    def forward(self, x: Tensor) -> VectorQuantizerOutput:
        temp = self._current_temperature()
        bsz, tsz, fsz = x.shape
        G, V = self.num_codebooks, self.num_codebook_entries
        logits = self.entry_proj(x.reshape(-1, fsz)).view(bsz * tsz * G, V)
        from fairseq2_b200.ops.wav2vec2 import gumbel_quantize, sample_gumbel_noise

        # one kernel: arg-max codes, soft probabilities, straight-through Gumbel sample and the code-book LOOKUP of
        # the selected entry (the dense formulation multiplies a [frames, G*V, 1] one-hot with the whole code book)
        noise = sample_gumbel_noise(tuple(logits.shape), logits.device) if self.training else None
        q, sel, prob_sum, hard_count = gumbel_quantize(logits, noise, self.entries.view(G * V, -1), G, temp, self.training)
        frames = max(bsz * tsz, 1)
        hard_probs = hard_count / frames
        code_perplexity = torch.exp(-torch.sum(hard_probs * torch.log(hard_probs + 1e-7), dim=-1)).sum()
        avg_probs = prob_sum / frames
        prob_perplexity = torch.exp(-torch.sum(avg_probs * torch.log(avg_probs + 1e-7), dim=-1)).sum()
        cb = torch.nn.functional.one_hot(sel.long().view(bsz * tsz, G), V).to(logits.dtype).view(bsz * tsz, G * V)
        return VectorQuantizerOutput(q.view(bsz, tsz, -1), cb, G, V, code_perplexity, prob_perplexity, temp)

    def _current_temperature(self) -> float:
        # `num_updates` lives on the device for checkpoints; reading it every step would stall the host until the
        # whole forward pass has run. A host-side mirror is read instead and refreshed whenever the buffer may have
        # changed behind our back (first use, checkpoint load, reset, a move to another device).
        key = (self.num_updates.data_ptr(), self.num_updates._version)
        if getattr(self, "_updates_key", None) != key:
            self._updates_host = int(self.num_updates)
        temp = max(self.max_temp * self.temp_decay ** self._updates_host, self.min_temp)
        if self.training:
            self.num_updates.add_(1)
            self._updates_host += 1
        self._updates_key = (self.num_updates.data_ptr(), self.num_updates._version)
        return temp


def _init_entry_projection(proj: Linear) -> None:
    torch.nn.init.normal_(proj.weight, mean=0.0, std=1.0)
    if proj.bias is not None:
        torch.nn.init.zeros_(proj.bias)
