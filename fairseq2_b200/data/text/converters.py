"""Native string converters (cf. fairseq2 ``data/text/converters.py``)."""
from fairseq2_b200.data.data_pipeline import _n

StrSplitter = _n.StrSplitter
StrToIntConverter = _n.StrToIntConverter
StrToTensorConverter = _n.StrToTensorConverter
