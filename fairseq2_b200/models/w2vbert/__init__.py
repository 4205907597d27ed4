from fairseq2_b200.models.w2vbert.model import (W2VBERT_FAMILY, W2VBertConfig, W2VBertLoss, W2VBertModel,
                                                W2VBertOutput, create_w2vbert_model)
