from fairseq2_b200.models.wav2vec2.config import (WAV2VEC2_FAMILY, Wav2Vec2Config, Wav2Vec2EncoderConfig)
from fairseq2_b200.models.wav2vec2.factory import (Wav2Vec2EncoderFactory, Wav2Vec2Factory, create_wav2vec2_model)
from fairseq2_b200.models.wav2vec2.feature_extractor import (Wav2Vec2FbankFeatureExtractor, Wav2Vec2FeatureExtractor)
from fairseq2_b200.models.wav2vec2.frontend import Wav2Vec2Frontend
from fairseq2_b200.models.wav2vec2.interop import convert_wav2vec2_asr_state_dict, convert_wav2vec2_state_dict
from fairseq2_b200.models.wav2vec2.masker import Wav2Vec2Masker
from fairseq2_b200.models.wav2vec2.model import Wav2Vec2Features, Wav2Vec2Loss, Wav2Vec2Model, Wav2Vec2Output
from fairseq2_b200.models.wav2vec2.position_encoder import Wav2Vec2PositionEncoder, Wav2Vec2StackedPositionEncoder
from fairseq2_b200.models.wav2vec2.vector_quantizer import GumbelVectorQuantizer, VectorQuantizer, VectorQuantizerOutput
