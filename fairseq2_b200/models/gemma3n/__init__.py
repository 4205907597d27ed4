from fairseq2_b200.models.gemma3n.config import GEMMA3N_FAMILY, Gemma3nConfig
from fairseq2_b200.models.gemma3n.factory import create_gemma3n_model, gemma3n_wrap_policy
from fairseq2_b200.models.gemma3n.interop import convert_gemma3n_state_dict, export_gemma3n_to_hg
from fairseq2_b200.models.gemma3n.model import Gemma3nModel

__all__ = ["GEMMA3N_FAMILY", "Gemma3nConfig", "Gemma3nModel", "convert_gemma3n_state_dict", "create_gemma3n_model",
           "export_gemma3n_to_hg", "gemma3n_wrap_policy"]
