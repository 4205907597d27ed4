from fairseq2_b200.models.transformer_lm.decoder import (StandardTransformerLMDecoder, TransformerLMDecoder,
                                                          TransformerLMDecoderLayerHook)
from fairseq2_b200.models.transformer_lm.decoder_layer import (StandardTransformerLMDecoderLayer,
                                                                TransformerLMDecoderLayer)
from fairseq2_b200.models.transformer_lm.model import TransformerLM
