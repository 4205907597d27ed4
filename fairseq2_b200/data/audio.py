"""Audio decoding and filter bank features (native; cf. fairseq2 ``data/audio.py``).
This build decodes RIFF/WAVE (PCM and float); other containers need libsndfile,
which is not part of the image."""
from fairseq2_b200.data.data_pipeline import _n

AudioDecoder = _n.AudioDecoder
WaveformToFbankConverter = _n.WaveformToFbankConverter
