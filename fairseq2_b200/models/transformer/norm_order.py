"""Where layer normalisation sits in a transformer layer
(cf. fairseq2 ``models/transformer/norm_order.py``)."""
from enum import Enum


class TransformerNormOrder(Enum):
    POST = 0
    PRE = 1
    PRE_WITH_NORMFORMER = 2
