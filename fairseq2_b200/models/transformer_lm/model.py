"""Decoder-only language model (cf. fairseq2 ``models/transformer_lm/model.py:25-215``).

With ``targets`` the output projection and the cross-entropy run as the fused,
chunked kernel pipeline of ``ops.cross_entropy`` -- the full ``[T, V]`` logits
are never resident -- unless logits are requested or label smoothing is on.
"""
from __future__ import annotations

from typing import Literal

from torch import Tensor

from fairseq2_b200.models.clm import CausalLM
from fairseq2_b200.models.transformer.frontend import TransformerFrontend
from fairseq2_b200.models.transformer_lm.decoder import TransformerLMDecoder
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.functional import cross_entropy
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, Projection, TiedProjection
from fairseq2_b200.ops.cross_entropy import fused_linear_cross_entropy


def _widen_batch(seqs: Tensor, layout: BatchLayout, targets: Tensor | None, target_mask: Tensor | None, pad: int,
                 pad_idx: int | None):  # type: ignore[no-untyped-def]
    """``pad`` more positions at the end of the token dimension: padding in the layout, masked out of the loss."""
    import torch
    import torch.nn.functional as F

    fill = pad_idx if pad_idx is not None else 0
    seqs = F.pad(seqs, (0, pad), value=fill)
    if layout.packed:
        layout = BatchLayout((seqs.shape[-1],), list(layout.seq_lens), packed=True, device=seqs.device)
    else:
        layout = BatchLayout(tuple(seqs.shape[:2]), list(layout.seq_lens), device=seqs.device)
    if targets is not None:
        if target_mask is None:
            target_mask = torch.ones(targets.shape, device=targets.device, dtype=torch.bool)
        targets = F.pad(targets, (0, pad), value=fill)
        target_mask = F.pad(target_mask, (0, pad), value=0)
    return seqs, layout, targets, target_mask


class TransformerLM(CausalLM):
    def __init__(self, model_dim: int, decoder_frontend: TransformerFrontend, decoder: TransformerLMDecoder,
                 final_proj: Projection, pad_idx: int | None, max_seq_len: int) -> None:
        super().__init__(max_seq_len)
        self.model_dim = model_dim
        self.decoder_frontend, self.decoder, self.final_proj = decoder_frontend, decoder, final_proj
        self.pad_idx = pad_idx

    def forward(self, seqs, seqs_layout, targets=None, *, state_bag=None, label_smoothing=0.0, target_mask=None,
                reduction="sum", return_logits=False):  # type: ignore[override]
        num_tokens = seqs.shape[-1]
        pad = self._sequence_parallel_padding(num_tokens) if state_bag is None else 0
        if pad:
            # token-sharded activations need a token count that the tensor-parallel ranks can split evenly: the
            # batch is widened by up to size - 1 padding positions that no sequence owns and no target counts
            seqs, seqs_layout, targets, target_mask = _widen_batch(seqs, seqs_layout, targets, target_mask, pad,
                                                                   self.pad_idx)
        seqs, seqs_layout = self.decoder_frontend(seqs, seqs_layout, state_bag=state_bag)
        out = self.decoder(seqs, seqs_layout, state_bag=state_bag)
        del seqs
        if targets is None:
            logits = self.final_proj(out)
            return logits[..., :num_tokens, :] if pad else logits
        if not return_logits:
            return self.compute_fused_loss(out, targets, label_smoothing=label_smoothing, target_mask=target_mask,
                                           reduction=reduction)
        logits = self.final_proj(out)
        loss = self.compute_loss(logits, targets, label_smoothing=label_smoothing, target_mask=target_mask,
                                 reduction=reduction)
        return loss, (logits[..., :num_tokens, :] if pad else logits)

    def _sequence_parallel_padding(self, num_tokens: int) -> int:
        if not getattr(self, "tp_sequence_parallel", False):
            return 0
        gang = getattr(self.final_proj, "gang", None)
        size = gang.size if gang is not None else 1
        return (-num_tokens) % size

    def compute_loss(self, logits: Tensor, targets: Tensor, *, label_smoothing: float = 0.0,
                     target_mask: Tensor | None = None, reduction: Literal["sum", "mean"] = "sum") -> Tensor:
        return cross_entropy(logits, targets, self.pad_idx, label_smoothing=label_smoothing, target_mask=target_mask,
                             reduction=reduction)

    def compute_fused_loss(self, decoder_output: Tensor, targets: Tensor, *, label_smoothing: float = 0.0,
                           target_mask: Tensor | None = None, reduction: Literal["sum", "mean"] = "sum") -> Tensor:
        fp = self.final_proj
        if label_smoothing == 0.0 and isinstance(fp, (Linear, TiedProjection)) and fp.bias is None:
            return fused_linear_cross_entropy(decoder_output, fp.weight, targets, target_mask=target_mask,
                                              pad_idx=self.pad_idx, reduction=reduction)
        if (label_smoothing == 0.0 and isinstance(fp, ColumnShardedLinear) and fp.bias is None and fp.gang.size > 1
                and fp.gather_output):
            # vocabulary-parallel output projection: every rank scores its slice of the vocabulary and only three
            # numbers per token cross the tensor-parallel gang; the [T, V] logits are never gathered
            from fairseq2_b200.ops.cross_entropy import vocab_parallel_linear_cross_entropy
            from fairseq2_b200.ops.tensor_parallel import all_gather_seq, reduce_on_backward

            h = decoder_output
            if fp.sequence_parallel:
                h = all_gather_seq(h, fp.gang, dim=-2)     # backward: reduce-scatter of the per-rank partial dh
            return vocab_parallel_linear_cross_entropy(h, fp.weight, targets, fp.gang, target_mask=target_mask,
                                                       pad_idx=self.pad_idx, reduction=reduction,
                                                       reduce_input_grad=not fp.sequence_parallel)
        return self.compute_loss(fp(decoder_output), targets, label_smoothing=label_smoothing,
                                 target_mask=target_mask, reduction=reduction)

    def extra_repr(self) -> str:
        return f"model_dim={self.model_dim}, pad_idx={self.pad_idx}, max_seq_len={self.max_seq_len}"
