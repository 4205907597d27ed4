"""wav2vec 2.0 self-supervised model (cf. fairseq2 ``models/wav2vec2/model.py:34-417``): masked frames of the
transformer output are contrasted against quantised targets and sampled distractors."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor
from torch.nn import Module
from torch.nn.functional import cross_entropy

from fairseq2_b200.models.transformer.encoder import TransformerEncoder
from fairseq2_b200.models.wav2vec2.frontend import Wav2Vec2Frontend
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker
from fairseq2_b200.models.wav2vec2.vector_quantizer import VectorQuantizer, VectorQuantizerOutput
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.typing import DataType, Device


@dataclass
class Wav2Vec2Features:
    seqs: Tensor
    seqs_layout: BatchLayout
    targets: Tensor
    temporal_mask: Tensor
    raw: Tensor


@dataclass
class Wav2Vec2Output:
    logits: Tensor
    """``(N, S_masked, 1 + num_distractors)``; index 0 is the true target."""
    quantized_targets: Tensor
    num_targets: int
    temporal_mask: Tensor
    quantizer_output: VectorQuantizerOutput
    encoder_output: Tensor
    encoder_output_layout: BatchLayout
    raw_features: Tensor
    contrastive_loss: Tensor | None = None
    """Summed cross entropy of ``logits`` against index 0, produced together with the logits by the fused kernel."""


@dataclass
class Wav2Vec2Loss:
    aggregate: Tensor
    contrastive: Tensor
    diversity: Tensor
    features_penalty: Tensor


class Wav2Vec2Model(Module):
    def __init__(self, model_dim: int, encoder_frontend: Wav2Vec2Frontend, encoder: TransformerEncoder,
                 masker: Wav2Vec2Masker, quantizer: VectorQuantizer, final_dim: int, *, final_proj_bias: bool = True,
                 num_distractors: int = 100, logit_temp: float = 0.1, quantizer_encoder_grad: bool = True,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__()
        self.model_dim = model_dim
        self.encoder_frontend, self.encoder, self.masker, self.quantizer = encoder_frontend, encoder, masker, quantizer
        self.quantizer_encoder_grad = quantizer_encoder_grad
        self.final_proj = Linear(model_dim, final_dim, final_proj_bias, device=device, dtype=dtype)
        self.final_target_proj = Linear(quantizer.output_dim, final_dim, bias=True, device=device, dtype=dtype)
        self.num_distractors, self.logit_temp = num_distractors, logit_temp

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, diversity_weight: float = 0.1,
                features_penalty_weight: float = 10.0) -> tuple[Wav2Vec2Loss, Wav2Vec2Output]:
        features = self.extract_features(seqs, seqs_layout)
        output = self.quantize_and_contrast(features)
        return self.compute_loss(output, diversity_weight=diversity_weight,
                                 features_penalty_weight=features_penalty_weight), output

    def extract_features(self, seqs: Tensor, seqs_layout: BatchLayout) -> Wav2Vec2Features:
        f = self.run_frontend(seqs, seqs_layout)
        f.seqs = self.encoder(f.seqs, f.seqs_layout)
        return f

    def run_frontend(self, seqs: Tensor, seqs_layout: BatchLayout) -> Wav2Vec2Features:
        fe = self.encoder_frontend
        seqs, seqs_layout, raw = fe.extract_features(seqs, seqs_layout)
        targets = seqs.clone() if self.quantizer_encoder_grad else seqs.detach().clone()
        if fe.first_pass_dropout is not None:
            targets = fe.first_pass_dropout(targets)
        seqs, mask = fe.process_features(seqs, seqs_layout, self.masker)
        assert mask is not None
        targets = Wav2Vec2Masker.extract_masked_elements(targets, mask)
        return Wav2Vec2Features(seqs, seqs_layout, targets, mask, raw)

    def quantize_and_contrast(self, f: Wav2Vec2Features) -> Wav2Vec2Output:
        seqs = self.final_proj(Wav2Vec2Masker.extract_masked_elements(f.seqs, f.temporal_mask))
        q = self.quantizer(f.targets)
        targets = self.final_target_proj(q.quantized_vectors)
        n, s, m = targets.shape
        from fairseq2_b200.ops.wav2vec2 import contrastive_logits_and_loss

        # logits and loss in one pass over index-given distractors; the [N, S, K, M] gather is never built
        idx = self._sample_distractor_indices(n, s, targets.device)
        logits, loss = contrastive_logits_and_loss(seqs.reshape(n * s, m), targets.reshape(n * s, m),
                                                   idx.view(n * s, -1), self.logit_temp)
        return Wav2Vec2Output(logits.view(n, s, -1), targets, n * s, f.temporal_mask, q, f.seqs, f.seqs_layout, f.raw,
                              contrastive_loss=loss)

    def _sample_distractor_indices(self, n: int, s: int, dev: torch.device) -> Tensor:
        """For every masked step, the rows (in the flattened ``[N * S, M]`` targets) of ``num_distractors`` other
        masked steps of the same utterance."""
        own = torch.arange(s, device=dev).repeat_interleave(self.num_distractors)
        rnd = torch.randint(0, max(s - 1, 1), (n, s * self.num_distractors), device=dev)
        rnd = rnd + (rnd >= own)                                      # skip the step itself
        if s == 1:
            rnd = torch.zeros_like(rnd)
        rnd = rnd + torch.arange(n, device=dev).unsqueeze(1) * s
        return rnd.view(n, s, self.num_distractors).to(torch.int32)

    def _sample_distractors(self, targets: Tensor) -> Tensor:
        n, s, m = targets.shape
        idx = self._sample_distractor_indices(n, s, targets.device)
        return targets.reshape(-1, m)[idx.view(-1).long()].view(n, s, self.num_distractors, m)

    def _compute_logits(self, seqs: Tensor, targets: Tensor, distractors: Tensor) -> Tensor:
        seqs, targets = seqs.unsqueeze(2), targets.unsqueeze(2)
        candidates = torch.cat([targets, distractors], dim=2)
        logits = torch.cosine_similarity(seqs.float(), candidates.float(), dim=-1)
        if self.logit_temp != 1.0:
            logits = logits / self.logit_temp
        same = (targets == distractors).all(-1)
        if same.any():
            logits[:, :, 1:][same] = float("-inf")
        return logits

    def compute_loss(self, output: Wav2Vec2Output, *, diversity_weight: float = 0.1,
                     features_penalty_weight: float = 10.0) -> Wav2Vec2Loss:
        logits = output.logits
        n, s, c = logits.shape
        if output.contrastive_loss is not None:
            contrastive = output.contrastive_loss
        else:
            flat = logits.transpose(0, 1).reshape(-1, c).float()
            contrastive = cross_entropy(flat, flat.new_zeros((n * s,), dtype=torch.int64), reduction="sum")
        entries = self.quantizer.num_codebooks * self.quantizer.num_codebook_entries  # type: ignore[attr-defined]
        diversity = (entries - output.quantizer_output.prob_perplexity) / entries * (n * s)
        penalty = output.raw_features.float().pow(2).mean() * (n * s)
        agg = contrastive + diversity_weight * diversity + features_penalty_weight * penalty
        return Wav2Vec2Loss(agg, contrastive, diversity, penalty)

    def extra_repr(self) -> str:
        return (f"model_dim={self.model_dim}, quantizer_encoder_grad={self.quantizer_encoder_grad}, "
                f"num_distractors={self.num_distractors}, logit_temp={self.logit_temp:G}")
