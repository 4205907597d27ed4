from fairseq2_b200.models.nllb.config import NLLB_FAMILY, NllbConfig
from fairseq2_b200.models.nllb.factory import create_nllb_model
from fairseq2_b200.models.nllb.interop import convert_nllb_state_dict
