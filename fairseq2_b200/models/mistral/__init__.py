from fairseq2_b200.models.mistral.config import MISTRAL_FAMILY, MistralConfig
from fairseq2_b200.models.mistral.factory import create_mistral_model
from fairseq2_b200.models.mistral.interop import convert_mistral_state_dict, export_mistral_to_hg
