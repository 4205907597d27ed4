from fairseq2_b200.models.jepa.model import (JEPA_CLASSIFIER_FAMILY, JEPA_FAMILY, AttentivePooler,
                                             CrossAttentionDecoderLayer, JepaClassifierConfig, JepaClassifierModel,
                                             JepaConfig, JepaEncoderConfig, JepaModel, convert_jepa_state_dict,
                                             create_jepa_classifier_model, create_jepa_model)
