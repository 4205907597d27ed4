from fairseq2_b200.models.s2t_transformer.config import (S2T_CONFORMER_FAMILY, S2T_TRANSFORMER_FAMILY,
                                                         S2TConformerConfig, S2TTransformerConfig)
from fairseq2_b200.models.s2t_transformer.factory import create_s2t_conformer_model, create_s2t_transformer_model
from fairseq2_b200.models.s2t_transformer.frontend import Conv1dFbankSubsampler, S2TTransformerFrontend
from fairseq2_b200.models.s2t_transformer.interop import convert_s2t_state_dict
