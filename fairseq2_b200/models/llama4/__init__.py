from fairseq2_b200.models.llama4.config import LLAMA4_FAMILY, Llama4Config, Llama4ExpertsConfig
from fairseq2_b200.models.llama4.factory import Llama4Factory, create_llama4_model
from fairseq2_b200.models.llama4.interop import convert_llama4_state_dict
