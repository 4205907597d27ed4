"""Builds wav2vec 2.0 ASR models (cf. fairseq2 ``models/wav2vec2/asr/factory.py:26-96``)."""
from __future__ import annotations

from fairseq2_b200.models.wav2vec2.asr.config import Wav2Vec2AsrConfig
from fairseq2_b200.models.wav2vec2.asr.model import Wav2Vec2AsrModel
from fairseq2_b200.models.wav2vec2.factory import Wav2Vec2EncoderFactory
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker


def create_wav2vec2_asr_model(config: Wav2Vec2AsrConfig, gangs: object | None = None) -> Wav2Vec2AsrModel:
    c = config
    ef = Wav2Vec2EncoderFactory(c.encoder_config)
    masker = None
    if c.use_masking:
        masker = Wav2Vec2Masker(c.encoder_config.model_dim, c.temporal_mask_span_len, c.max_temporal_mask_prob,
                                c.min_num_temporal_mask_spans, c.spatial_mask_span_len, c.max_spatial_mask_prob,
                                c.min_num_spatial_mask_spans)
    return Wav2Vec2AsrModel(c.encoder_config.model_dim, ef.create_encoder_frontend(), ef.create_encoder(),
                            c.target_vocab_size, masker=masker, final_dropout_p=c.final_dropout_p)
