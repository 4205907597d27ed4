"""w2v-BERT (cf. fairseq2 ``models/w2vbert/config.py:22-121``, ``w2vbert/model.py:30-214``, ``w2vbert/factory.py``):
a Conformer wav2vec 2.0 whose lower layers feed the contrastive objective while the output of the full stack
predicts the quantiser's code indices at the masked steps (masked prediction)."""
from __future__ import annotations

from dataclasses import dataclass, field

from torch import Tensor
from torch.nn import Module
from torch.nn.functional import cross_entropy

from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.wav2vec2.config import Wav2Vec2Config, Wav2Vec2EncoderConfig
from fairseq2_b200.models.wav2vec2.factory import Wav2Vec2Factory
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker
from fairseq2_b200.models.wav2vec2.model import Wav2Vec2Loss, Wav2Vec2Model, Wav2Vec2Output
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.runtime.config_registry import ConfigRegistrar
from fairseq2_b200.utils.validation import ValidationResult

W2VBERT_FAMILY = "w2vbert"


def _w2v2_600m() -> Wav2Vec2Config:
    e = Wav2Vec2EncoderConfig(
        model_dim=1024, max_seq_len=4096, feature_dim=160, use_fbank=True, first_pass_dropout_p=0.0,
        layer_norm_features=False, feature_extractor_layer_descs=[], feature_extractor_bias=False,
        feature_extractor_layer_norm_convs=False, feature_grad_scale=1.0, num_fbank_channels=80, fbank_stride=2,
        sample_fbank_every_k=1, pos_encoder_type="relative", pos_encoder_depth=0, pos_conv_kernel_size=0,
        num_pos_conv_groups=0, use_conformer=True, num_encoder_layers=24, num_encoder_attn_heads=16,
        ffn_inner_dim=4096, dropout_p=0.0, attn_dropout_p=0.0, layer_drop_p=0.0,
        norm_order=TransformerNormOrder.POST, depthwise_conv_kernel_size=31)
    return Wav2Vec2Config(encoder_config=e, final_dim=768, final_proj_bias=True, temporal_mask_span_len=10,
                          max_temporal_mask_prob=0.65, min_num_temporal_mask_spans=2, spatial_mask_span_len=10,
                          max_spatial_mask_prob=0.0, min_num_spatial_mask_spans=2, quantized_dim=1024, num_codebooks=1,
                          num_codebook_entries=1024, codebook_sampling_temperature=(2.0, 0.1, 0.999995),
                          num_distractors=100, logit_temp=0.1)


@dataclass(kw_only=True)
class W2VBertConfig:
    w2v2_config: Wav2Vec2Config = field(default_factory=_w2v2_600m)
    num_bert_encoder_layers: int = 16
    """The top layers of the encoder that only serve masked prediction."""
    num_target_codebooks: int = 1

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        e = self.w2v2_config.encoder_config
        if e.layer_drop_p != 0.0:
            r.add_error("`w2v2_config.encoder_config.layer_drop_p` must be 0.0 since w2v-BERT does not support LayerDrop.")
        if self.num_bert_encoder_layers >= e.num_encoder_layers:
            r.add_error(f"`num_bert_encoder_layers` must be less than the number of encoder layers ({e.num_encoder_layers}).")
        if self.num_target_codebooks > self.w2v2_config.num_codebooks:
            r.add_error(f"`num_target_codebooks` must not exceed `w2v2_config.num_codebooks` ({self.w2v2_config.num_codebooks}).")
        return r


arch = ConfigRegistrar(W2VBertConfig)


@arch("600m")
def w2vbert_600m() -> W2VBertConfig:
    return W2VBertConfig()


@arch("300m")
def w2vbert_300m() -> W2VBertConfig:
    c = W2VBertConfig()
    c.w2v2_config.encoder_config.num_encoder_layers = 12
    c.num_bert_encoder_layers = 8
    return c


@arch("tiny")
def w2vbert_tiny() -> W2VBertConfig:
    c = W2VBertConfig()
    e = c.w2v2_config.encoder_config
    e.model_dim, e.feature_dim, e.num_fbank_channels, e.max_seq_len = 64, 32, 16, 512
    e.num_encoder_layers, e.num_encoder_attn_heads, e.ffn_inner_dim, e.depthwise_conv_kernel_size = 3, 4, 128, 7
    w = c.w2v2_config
    w.final_dim, w.quantized_dim, w.num_codebook_entries, w.num_distractors, w.temporal_mask_span_len = 32, 32, 16, 10, 3
    c.num_bert_encoder_layers = 1
    return c


@dataclass
class W2VBertOutput:
    w2v2_output: Wav2Vec2Output
    bert_logits: Tensor
    """``(N·S_masked, V, G_target)``."""
    bert_targets: Tensor
    """``(N·S_masked, G_target)``."""


@dataclass
class W2VBertLoss:
    aggregate: Tensor
    bert: Tensor
    w2v2: Wav2Vec2Loss


class W2VBertModel(Module):
    def __init__(self, w2v2_model: Wav2Vec2Model, num_bert_encoder_layers: int, *, num_target_codebooks: int = 1) -> None:
        super().__init__()
        self.model_dim = w2v2_model.model_dim
        self.w2v2_model = w2v2_model
        self.num_bert_encoder_layers = num_bert_encoder_layers
        self.num_target_codebooks = num_target_codebooks
        entries = w2v2_model.quantizer.num_codebook_entries  # type: ignore[attr-defined]
        self.final_bert_proj = Linear(self.model_dim, entries * num_target_codebooks, bias=True)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, bert_weight: float = 1.0,
                bert_label_smoothing: float = 0.0, w2v2_weight: float = 1.0, w2v2_diversity_weight: float = 0.1,
                w2v2_features_penalty_weight: float = 10.0) -> tuple[W2VBertLoss, W2VBertOutput]:
        w = self.w2v2_model
        feats = w.run_frontend(seqs, seqs_layout)
        tap: dict[str, Tensor] = {}

        def hook(layer_idx: int, out: Tensor, layout: BatchLayout, num_layers: int) -> bool:
            if layer_idx == num_layers - self.num_bert_encoder_layers - 1:
                tap["seqs"] = out                      # output of the contrastive part of the stack
            return True

        handle = w.encoder.register_layer_hook(hook)
        try:
            encoder_output = w.encoder(feats.seqs, feats.seqs_layout)
        finally:
            handle.remove()
        feats.seqs = tap["seqs"]
        w2v2_out = w.quantize_and_contrast(feats)
        masked = Wav2Vec2Masker.extract_masked_elements(encoder_output, feats.temporal_mask)
        entries = w.quantizer.num_codebook_entries  # type: ignore[attr-defined]
        logits = self.final_bert_proj(masked).view(-1, entries, self.num_target_codebooks)
        G = w.quantizer.num_codebooks  # type: ignore[attr-defined]
        n, s = w2v2_out.quantizer_output.quantized_vectors.shape[:2]
        cb = w2v2_out.quantizer_output.cb.view(n * s * G, -1)
        targets = cb.argmax(dim=-1).view(-1, G)[..., : self.num_target_codebooks].detach()
        out = W2VBertOutput(w2v2_out, logits, targets)
        bert = cross_entropy(logits.float(), targets, reduction="sum", label_smoothing=bert_label_smoothing)
        w2 = w.compute_loss(w2v2_out, diversity_weight=w2v2_diversity_weight,
                            features_penalty_weight=w2v2_features_penalty_weight)
        return W2VBertLoss(bert_weight * bert + w2v2_weight * w2.aggregate, bert, w2), out

    def extra_repr(self) -> str:
        return (f"model_dim={self.model_dim}, num_bert_encoder_layers={self.num_bert_encoder_layers}, "
                f"num_target_codebooks={self.num_target_codebooks}")


def create_w2vbert_model(config: W2VBertConfig, gangs: object | None = None) -> W2VBertModel:
    w2v2 = Wav2Vec2Factory(config.w2v2_config).create_model()
    return W2VBertModel(w2v2, config.num_bert_encoder_layers, num_target_codebooks=config.num_target_codebooks)
