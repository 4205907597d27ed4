"""WAV / AIFF / AIFF-C / AU decoding of the native ``AudioDecoder``: files are assembled byte by byte here (and, where
the standard library still ships a writer, by it), the decoded samples must equal the source exactly."""
from __future__ import annotations

import io
import struct
import warnings

import numpy as np
import pytest
import torch

from fairseq2_b200.data.audio import AudioDecoder
from fairseq2_b200.data.data_pipeline import MemoryBlock

_RNG = np.random.default_rng(0)
_PCM16 = _RNG.integers(-32768, 32767, size=(100, 2), dtype=np.int16)


def _decode(blob: bytes, **kwargs):  # type: ignore[no-untyped-def]
    return AudioDecoder(**kwargs)(MemoryBlock(blob))


def _wav(tag: int, bits: int, channels: int, rate: int, data: bytes, extensible: bool = False) -> bytes:
    block = channels * bits // 8
    if extensible:
        fmt = struct.pack("<HHIIHHHHIH14s", 0xFFFE, channels, rate, rate * block, block, bits, 22, bits, 3, tag,
                          b"\x00\x00\x00\x00\x10\x00\x80\x00\x00\xaa\x00\x38\x9b\x71")
    else:
        fmt = struct.pack("<HHIIHH", tag, channels, rate, rate * block, block, bits)
    body = b"WAVE" + b"fmt " + struct.pack("<I", len(fmt)) + fmt + b"LIST" + struct.pack("<I", 3) + b"abc\x00"
    body += b"data" + struct.pack("<I", len(data)) + data
    return b"RIFF" + struct.pack("<I", len(body)) + body


def _extended(rate: float) -> bytes:
    """80-bit IEEE extended, as AIFF stores the sample rate."""
    mantissa, exponent = np.frexp(rate)
    return struct.pack(">HQ", int(exponent) - 1 + 16383, int(mantissa * 2 ** 64))


def _aiff(bits: int, channels: int, rate: float, data: bytes, compression: bytes | None = None, offset: int = 0) -> bytes:
    frames = len(data) // (channels * ((bits + 7) // 8))
    comm = struct.pack(">hIh", channels, frames, bits) + _extended(rate)
    if compression is not None:
        comm += compression + b"\x00\x00"
    ssnd = struct.pack(">II", offset, 0) + b"\x00" * offset + data
    chunks = b"COMM" + struct.pack(">I", len(comm)) + comm + b"SSND" + struct.pack(">I", len(ssnd)) + ssnd
    if len(ssnd) & 1:
        chunks += b"\x00"
    form = (b"AIFC" if compression is not None else b"AIFF") + chunks
    return b"FORM" + struct.pack(">I", len(form)) + form


def _au(encoding: int, channels: int, rate: int, data: bytes, unknown_size: bool = False) -> bytes:
    return b".snd" + struct.pack(">IIIII", 28, 0xFFFFFFFF if unknown_size else len(data), encoding, rate, channels) + b"info" + data


def test_wav_integer_widths_are_exact() -> None:
    out = _decode(_wav(1, 16, 2, 22050, _PCM16.tobytes()))
    assert out["format"] == "WAV/PCM_16" and out["sample_rate"] == 22050.0 and out["waveform"].dtype == torch.int16
    assert torch.equal(out["waveform"], torch.from_numpy(_PCM16))
    p32 = _RNG.integers(-2 ** 31, 2 ** 31 - 1, size=(50,), dtype=np.int32)
    out = _decode(_wav(1, 32, 1, 48000, p32.tobytes()))
    assert out["format"] == "WAV/PCM_32" and out["waveform"].dtype == torch.int32
    assert torch.equal(out["waveform"], torch.from_numpy(p32))             # no float round trip in between
    p24 = _RNG.integers(-2 ** 23, 2 ** 23 - 1, size=(60,), dtype=np.int32)
    raw = b"".join(int(v).to_bytes(3, "little", signed=True) for v in p24)
    out = _decode(_wav(1, 24, 1, 16000, raw, extensible=True))
    assert out["format"] == "WAV/PCM_24" and torch.equal(out["waveform"], torch.from_numpy(p24))
    as_float = _decode(_wav(1, 24, 1, 16000, raw), dtype=torch.float64)["waveform"]
    assert torch.equal(as_float, torch.from_numpy(p24).double() / 2 ** 23)
    u8 = _RNG.integers(0, 255, size=(30,), dtype=np.uint8)
    out = _decode(_wav(1, 8, 1, 8000, u8.tobytes()))
    assert torch.equal(out["waveform"].int(), torch.from_numpy(u8.astype(np.int32) - 128))
    keep = _decode(_wav(1, 16, 1, 8000, _PCM16[:, 0].tobytes()), keepdim=True)["waveform"]
    assert keep.shape == (100, 1)


def test_wav_float_and_double() -> None:
    f32 = _RNG.standard_normal((40, 2)).astype(np.float32)
    out = _decode(_wav(3, 32, 2, 48000, f32.tobytes()))
    assert out["format"] == "WAV/FLOAT" and torch.equal(out["waveform"], torch.from_numpy(f32))
    f64 = _RNG.standard_normal((40, 2))
    out = _decode(_wav(3, 64, 2, 48000, f64.tobytes()), dtype=torch.float64)
    assert out["format"] == "WAV/DOUBLE" and torch.equal(out["waveform"], torch.from_numpy(f64))


def test_aiff_big_endian_little_endian_and_float() -> None:
    out = _decode(_aiff(16, 2, 44100.0, _PCM16.byteswap().tobytes(), offset=4))
    assert out["format"] == "AIFF/PCM_16" and out["sample_rate"] == 44100.0
    assert torch.equal(out["waveform"], torch.from_numpy(_PCM16))
    out = _decode(_aiff(16, 2, 22050.0, _PCM16.tobytes(), compression=b"sowt"))
    assert torch.equal(out["waveform"], torch.from_numpy(_PCM16))
    f32 = _RNG.standard_normal((31, 1)).astype(np.float32)
    out = _decode(_aiff(32, 1, 96000.0, f32.byteswap().tobytes(), compression=b"fl32"))
    assert out["format"] == "AIFF/FLOAT" and out["sample_rate"] == 96000.0
    assert torch.equal(out["waveform"], torch.from_numpy(f32[:, 0]))
    p24 = _RNG.integers(-2 ** 23, 2 ** 23 - 1, size=(33,), dtype=np.int32)
    raw = b"".join(int(v).to_bytes(3, "big", signed=True) for v in p24)
    assert torch.equal(_decode(_aiff(24, 1, 8000.0, raw))["waveform"], torch.from_numpy(p24))
    with pytest.raises(ValueError, match="compression type"):
        _decode(_aiff(16, 1, 8000.0, b"\x00" * 8, compression=b"ima4"))


def test_au_encodings() -> None:
    out = _decode(_au(3, 2, 16000, _PCM16.byteswap().tobytes(), unknown_size=True))
    assert out["format"] == "AU/PCM_16" and out["sample_rate"] == 16000.0
    assert torch.equal(out["waveform"], torch.from_numpy(_PCM16))
    f64 = _RNG.standard_normal((20,))
    out = _decode(_au(7, 1, 8000, f64.byteswap().tobytes()), dtype=torch.float64)
    assert out["format"] == "AU/DOUBLE" and torch.equal(out["waveform"], torch.from_numpy(f64))
    i8 = _RNG.integers(-128, 127, size=(20,), dtype=np.int8)
    assert torch.equal(_decode(_au(2, 1, 8000, i8.tobytes()))["waveform"].int(), torch.from_numpy(i8.astype(np.int32)))
    with pytest.raises(ValueError, match="encoding"):
        _decode(_au(23, 1, 8000, b"\x00" * 8))


def test_companded_samples() -> None:
    codes = bytes(range(256))
    # G.711 anchor values: the largest magnitudes, and the two zero codes
    mu = _decode(_au(1, 1, 8000, codes))["waveform"]
    assert mu.dtype == torch.int16 and mu[0x00] == -32124 and mu[0x80] == 32124 and mu[0xFF] == 0 and mu[0x7F] == 0
    al = _decode(_au(27, 1, 8000, codes))["waveform"]
    assert al[0x2A] == -32256 and al[0xAA] == 32256 and al[0xD5] == 8 and al[0x55] == -8
    assert _decode(_wav(7, 8, 1, 8000, codes))["format"] == "WAV/ULAW"
    assert torch.equal(_decode(_wav(7, 8, 1, 8000, codes))["waveform"], mu)
    assert torch.equal(_decode(_wav(6, 8, 1, 8000, codes))["waveform"], al)
    assert torch.equal(_decode(_aiff(8, 1, 8000.0, codes, compression=b"alaw"))["waveform"], al)
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            import audioop
    except ImportError:
        return
    assert mu.tolist() == list(np.frombuffer(audioop.ulaw2lin(codes, 2), dtype=np.int16))
    assert al.tolist() == list(np.frombuffer(audioop.alaw2lin(codes, 2), dtype=np.int16))


def test_standard_library_writers_round_trip() -> None:
    class Keep(io.BytesIO):
        def close(self) -> None:
            pass

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            import aifc
            import sunau
        except ImportError:
            pytest.skip("the standard library of this interpreter has no AIFF / AU writers")
        buf = Keep()
        a = aifc.open(buf, "wb")
        a.setnchannels(2), a.setsampwidth(2), a.setframerate(44100)
        a.writeframes(_PCM16.byteswap().tobytes())
        a.close()
        assert torch.equal(_decode(buf.getvalue())["waveform"], torch.from_numpy(_PCM16))
        buf = Keep()
        u = sunau.open(buf, "wb")
        u.setnchannels(2), u.setsampwidth(2), u.setframerate(16000), u.setcomptype("NONE", "")
        u.writeframes(_PCM16.byteswap().tobytes())
        u.close()
        assert torch.equal(_decode(buf.getvalue())["waveform"], torch.from_numpy(_PCM16))


def test_broken_containers_are_refused() -> None:
    with pytest.raises(ValueError):
        _decode(b"RIFF" + struct.pack("<I", 4) + b"WAVE" + b"\x00" * 40)              # no fmt / data chunk
    with pytest.raises(ValueError):
        _decode(_wav(2, 4, 1, 8000, b"\x00" * 16))                                     # ADPCM
    with pytest.raises(ValueError):
        _decode(b"FORM" + struct.pack(">I", 4) + b"AIFF" + b"\x00" * 40)              # no COMM chunk
    with pytest.raises(ValueError):
        _decode(b"MThd" + b"\x00" * 60)                                                # not audio at all
    with pytest.raises(ValueError, match="Ogg"):
        _decode(b"OggS" + b"\x00" * 60)
    # a data chunk that claims more than the file holds is cut at the end of the file
    short = bytearray(_wav(1, 16, 1, 8000, _PCM16[:, 0].tobytes()))
    assert _decode(bytes(short[:-50]))["waveform"].shape == (75,)
