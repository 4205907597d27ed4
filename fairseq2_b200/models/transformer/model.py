"""Encoder-decoder Transformer (cf. fairseq2 ``models/transformer/model.py:24-260``).

In evaluation with a state bag the encoder output is computed once and cached
in the bag, so incremental decoding only runs the decoder."""
from __future__ import annotations

from typing import Literal

from torch import Tensor

from fairseq2_b200.models.seq2seq import Seq2SeqModel
from fairseq2_b200.models.transformer.decoder import TransformerDecoder
from fairseq2_b200.models.transformer.encoder import TransformerEncoder
from fairseq2_b200.models.transformer.frontend import TransformerFrontend
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.functional import cross_entropy
from fairseq2_b200.nn.incremental_state import IncrementalState, IncrementalStateBag
from fairseq2_b200.nn.projection import Linear, Projection, TiedProjection
from fairseq2_b200.ops.cross_entropy import fused_linear_cross_entropy


class _EncoderOutputState(IncrementalState):
    def __init__(self, encoder_output: Tensor, layout: BatchLayout) -> None:
        self.encoder_output, self.layout = encoder_output, layout

    def reorder(self, new_order: Tensor) -> None:
        self.encoder_output = self.encoder_output.index_select(0, new_order)
        lens = [self.layout.seq_lens[i] for i in new_order.tolist()]
        self.layout = BatchLayout(tuple(self.encoder_output.shape[:2]), lens, device=self.encoder_output.device)

    def size_bytes(self) -> int:
        return self.encoder_output.numel() * self.encoder_output.element_size()

    def capacity_bytes(self) -> int:
        return self.size_bytes()


class TransformerModel(Seq2SeqModel):
    def __init__(self, model_dim: int, encoder_frontend: TransformerFrontend, encoder: TransformerEncoder,
                 decoder_frontend: TransformerFrontend, decoder: TransformerDecoder, final_proj: Projection,
                 pad_idx: int | None, max_source_seq_len: int, max_target_seq_len: int) -> None:
        super().__init__(max_source_seq_len, max_target_seq_len)
        self.model_dim = model_dim
        self.encoder_frontend, self.encoder = encoder_frontend, encoder
        self.decoder_frontend, self.decoder = decoder_frontend, decoder
        self.final_proj = final_proj
        self.pad_idx = pad_idx

    def encode(self, source_seqs: Tensor, source_seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout]:
        seqs, layout = self.encoder_frontend(source_seqs, source_seqs_layout)
        return self.encoder(seqs, layout), layout

    def decode(self, target_seqs: Tensor, target_seqs_layout: BatchLayout, encoder_output: Tensor,
               encoder_output_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        seqs, layout = self.decoder_frontend(target_seqs, target_seqs_layout, state_bag=state_bag)
        return self.decoder(seqs, layout, encoder_output, encoder_output_layout, state_bag=state_bag)

    def forward(self, source_seqs, source_seqs_layout, target_seqs, target_seqs_layout, targets=None, *,  # type: ignore[override]
                state_bag=None, label_smoothing=0.0, target_mask=None, reduction="sum", return_logits=False):
        state = None
        caching = not self.training and state_bag is not None
        if caching:
            state = state_bag.maybe_get_state(self, _EncoderOutputState)
        if state is None:
            enc, enc_layout = self.encode(source_seqs, source_seqs_layout)
            if caching:
                state_bag.set_state(self, _EncoderOutputState(enc, enc_layout))
        else:
            enc, enc_layout = state.encoder_output, state.layout
        out = self.decode(target_seqs, target_seqs_layout, enc, enc_layout, state_bag=state_bag)
        if targets is None:
            return self.final_proj(out)
        fp = self.final_proj
        if (not return_logits and label_smoothing == 0.0 and isinstance(fp, (Linear, TiedProjection))
                and fp.bias is None):
            return fused_linear_cross_entropy(out, fp.weight, targets, target_mask=target_mask, pad_idx=self.pad_idx,
                                              reduction=reduction)
        logits = fp(out)
        loss = cross_entropy(logits, targets, self.pad_idx, label_smoothing=label_smoothing, target_mask=target_mask,
                             reduction=reduction)
        return (loss, logits) if return_logits else loss
