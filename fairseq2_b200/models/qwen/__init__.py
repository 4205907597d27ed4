from fairseq2_b200.models.qwen.config import QWEN_FAMILY, QwenConfig
from fairseq2_b200.models.qwen.factory import create_qwen_model
from fairseq2_b200.models.qwen.interop import convert_qwen_state_dict, export_qwen_to_hg
