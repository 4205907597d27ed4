from fairseq2_b200.models.llama.config import (LLAMA_FAMILY, LLaMAConfig, LLaMARoPEScaleConfig, get_llama_config)
from fairseq2_b200.models.llama.factory import LLaMAFactory, create_llama_model, init_llama_rope_freqs
