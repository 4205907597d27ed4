"""Image decoding (native PNG decoder over zlib; cf. fairseq2 ``data/image.py``)."""
from fairseq2_b200.data.data_pipeline import _n

ImageDecoder = _n.ImageDecoder
