from fairseq2_b200.models.olmo.config import OLMO_FAMILY, OLMOConfig, YaRNScaleConfig
from fairseq2_b200.models.olmo.factory import (OLMOTransformerLMDecoderLayer, YaRNRotaryEncoder, create_olmo_model,
                                               yarn_inv_freqs)
from fairseq2_b200.models.olmo.interop import convert_olmo_state_dict, export_olmo_to_hg
