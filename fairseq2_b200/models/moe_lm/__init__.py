from fairseq2_b200.models.moe_lm.config import MOE_LM_FAMILY, MoELMConfig
from fairseq2_b200.models.moe_lm.factory import MoELMFactory, MoETransformerLM, create_moe_lm_model
