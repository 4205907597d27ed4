"""Image decoding on the native runtime (cf. fairseq2 ``data/image.py``): ``ImageDecoder(device=None,
pin_memory=False)`` maps a ``MemoryBlock`` to ``{"image" [H, W, C], "channels", "height", "width", "bit_depth"}``
(PNG also ``"color_type"``). PNG: every colour type and bit depth, Adam7 interlacing, palette transparency; JPEG:
sequential and progressive. No codec library is needed besides zlib."""
from fairseq2_b200.data.data_pipeline import _n

ImageDecoder = _n.ImageDecoder
