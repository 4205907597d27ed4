from fairseq2_b200.models.wav2vec2.asr.config import WAV2VEC2_ASR_FAMILY, Wav2Vec2AsrConfig
from fairseq2_b200.models.wav2vec2.asr.factory import create_wav2vec2_asr_model
from fairseq2_b200.models.wav2vec2.asr.model import Wav2Vec2AsrModel
