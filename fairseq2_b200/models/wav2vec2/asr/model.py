"""wav2vec 2.0 fine-tuned with CTC (cf. fairseq2 ``models/wav2vec2/asr/model.py:30-174``)."""
from __future__ import annotations

import torch
from torch import Tensor
from torch.nn import Dropout
from torch.nn.functional import ctc_loss, log_softmax

from fairseq2_b200.models.asr import AsrModel
from fairseq2_b200.models.transformer.encoder import TransformerEncoder
from fairseq2_b200.models.wav2vec2.frontend import Wav2Vec2Frontend
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.typing import DataType, Device


def _init_final_projection(p: Linear) -> None:
    torch.nn.init.xavier_uniform_(p.weight)
    if p.bias is not None:
        torch.nn.init.zeros_(p.bias)


class Wav2Vec2AsrModel(AsrModel):
    def __init__(self, model_dim: int, encoder_frontend: Wav2Vec2Frontend, encoder: TransformerEncoder,
                 target_vocab_size: int, *, masker: Wav2Vec2Masker | None = None, final_dropout_p: float = 0.0,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__()
        self.model_dim = model_dim
        self.encoder_frontend, self.encoder, self.masker = encoder_frontend, encoder, masker
        self.final_dropout = Dropout(final_dropout_p) if final_dropout_p > 0.0 else None
        self.final_proj = Linear(model_dim, target_vocab_size, bias=True, init_fn=_init_final_projection,
                                 device=device, dtype=dtype)

    def forward(self, seqs, seqs_layout, targets=None, targets_layout=None, *, return_logits=False):  # type: ignore[override]
        fe = self.encoder_frontend
        seqs, layout, _ = fe.extract_features(seqs, seqs_layout)
        seqs, _ = fe.process_features(seqs, layout, self.masker if self.training else None)
        seqs = self.encoder(seqs, layout)
        if self.final_dropout is not None:
            seqs = self.final_dropout(seqs)
        logits = self.final_proj(seqs)
        if targets is None:
            return logits, layout
        if targets_layout is None:
            raise ValueError("`targets_layout` must be specified when `targets` is specified.")
        loss = self.compute_loss(logits, layout, targets, targets_layout)
        return (loss, logits, layout) if return_logits else loss

    @staticmethod
    def compute_loss(logits: Tensor, logits_layout: BatchLayout, targets: Tensor, targets_layout: BatchLayout) -> Tensor:
        """Sum-reduced CTC loss with blank index 0; log-probabilities in fp32, infinite losses zeroed."""
        lprobs = log_softmax(logits, dim=-1, dtype=torch.float32).transpose(0, 1)      # (S, N, V)
        return ctc_loss(lprobs, targets, logits_layout.seq_lens_pt, targets_layout.seq_lens_pt, reduction="sum",
                        zero_infinity=True)
