"""The native PNG decoder: every colour type and bit depth, Adam7 interlacing, all five scanline filters, palette
transparency, checksums. Files are written by a small encoder in this file (Pillow cannot write interlaced or
low-depth files on request); Pillow reading the same bytes is the second opinion."""
from __future__ import annotations

import io
import struct
import zlib

import numpy as np
import pytest
import torch

from fairseq2_b200.data.data_pipeline import MemoryBlock
from fairseq2_b200.data.image import ImageDecoder

_ADAM7 = [(0, 0, 8, 8), (4, 0, 8, 8), (0, 4, 4, 8), (2, 0, 4, 4), (0, 2, 2, 4), (1, 0, 2, 2), (0, 1, 1, 2)]
_CHANNELS = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}


def _chunk(kind: bytes, body: bytes) -> bytes:
    return struct.pack(">I", len(body)) + kind + body + struct.pack(">I", zlib.crc32(kind + body))


def _pack_rows(samples: np.ndarray, depth: int) -> list[bytes]:
    """``samples``: [h, w, c] unsigned; one packed scanline per row."""
    rows = []
    for row in samples:
        flat = row.reshape(-1)
        if depth == 16:
            rows.append(flat.astype(">u2").tobytes())
        elif depth == 8:
            rows.append(flat.astype(np.uint8).tobytes())
        else:
            bits = np.zeros(((len(flat) * depth + 7) // 8) * 8, dtype=np.uint8)
            for k in range(depth):
                bits[k::depth][: len(flat)] = (flat >> (depth - 1 - k)) & 1
            rows.append(np.packbits(bits).tobytes())
    return rows


def _filter(rows: list[bytes], bpp: int, rng: np.random.Generator) -> bytes:
    """Every row gets a random filter type; the arithmetic is the specification's."""
    out = bytearray()
    prev = bytes(len(rows[0])) if rows else b""
    for row in rows:
        kind = int(rng.integers(0, 5))
        cur = np.frombuffer(row, dtype=np.uint8).astype(np.int32)
        up = np.frombuffer(prev, dtype=np.uint8).astype(np.int32)
        left = np.concatenate([np.zeros(bpp, np.int32), cur[:-bpp]]) if len(cur) > bpp else np.zeros_like(cur)
        upleft = np.concatenate([np.zeros(bpp, np.int32), up[:-bpp]]) if len(up) > bpp else np.zeros_like(up)
        if kind == 0:
            pred = np.zeros_like(cur)
        elif kind == 1:
            pred = left
        elif kind == 2:
            pred = up
        elif kind == 3:
            pred = (left + up) // 2
        else:
            p = left + up - upleft
            pa, pb, pc = np.abs(p - left), np.abs(p - up), np.abs(p - upleft)
            pred = np.where((pa <= pb) & (pa <= pc), left, np.where(pb <= pc, up, upleft))
        out.append(kind)
        out += ((cur - pred) % 256).astype(np.uint8).tobytes()
        prev = row
    return bytes(out)


def _encode(samples: np.ndarray, depth: int, color: int, *, interlace: bool = False, palette: np.ndarray | None = None,
            trns: bytes | None = None, split_idat: int = 0, seed: int = 0) -> bytes:
    rng = np.random.default_rng(seed)
    h, w, c = samples.shape
    assert c == _CHANNELS[color]
    bpp = max(1, c * depth // 8)
    body = bytearray()
    if interlace:
        for x0, y0, dx, dy in _ADAM7:
            sub = samples[y0::dy, x0::dx]
            if sub.shape[0] and sub.shape[1]:
                body += _filter(_pack_rows(sub, depth), bpp, rng)
    else:
        body += _filter(_pack_rows(samples, depth), bpp, rng)
    data = zlib.compress(bytes(body), 6)
    out = b"\x89PNG\r\n\x1a\n" + _chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, depth, color, 0, 0, int(interlace)))
    out += _chunk(b"tEXt", b"Comment\x00made by the test")
    if palette is not None:
        out += _chunk(b"PLTE", palette.astype(np.uint8).tobytes())
    if trns is not None:
        out += _chunk(b"tRNS", trns)
    if split_idat:
        for i in range(0, len(data), split_idat):
            out += _chunk(b"IDAT", data[i:i + split_idat])
    else:
        out += _chunk(b"IDAT", data)
    return out + _chunk(b"IEND", b"")


def _decode(blob: bytes):  # type: ignore[no-untyped-def]
    return ImageDecoder()(MemoryBlock(blob))


def _unsigned(t: torch.Tensor) -> np.ndarray:
    a = t.numpy()
    return a.view(np.uint16) if a.dtype == np.int16 else a


@pytest.mark.parametrize("interlace", [False, True])
@pytest.mark.parametrize("color,depth", [(0, 1), (0, 2), (0, 4), (0, 8), (0, 16), (2, 8), (2, 16), (4, 8), (4, 16),
                                         (6, 8), (6, 16)])
def test_direct_colour_types(color: int, depth: int, interlace: bool) -> None:
    rng = np.random.default_rng(depth * 10 + color)
    for h, w in ((1, 1), (3, 5), (9, 17), (16, 8), (33, 31)):
        samples = rng.integers(0, 2 ** depth, size=(h, w, _CHANNELS[color]), dtype=np.uint32)
        blob = _encode(samples, depth, color, interlace=interlace, split_idat=64 if h > 8 else 0, seed=h)
        out = _decode(blob)
        got = _unsigned(out["image"])
        want = samples * 255 // (2 ** depth - 1) if depth < 8 else samples
        assert got.shape == (h, w, _CHANNELS[color]) and np.array_equal(got.astype(np.uint32), want), (h, w)
        assert out["bit_depth"] == depth and out["color_type"] == color and out["channels"] == _CHANNELS[color]
        assert out["height"] == h and out["width"] == w


def test_pillow_reads_the_same_pixels() -> None:
    PIL = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(5)
    for color, mode in ((0, "L"), (2, "RGB"), (6, "RGBA")):
        samples = rng.integers(0, 256, size=(21, 37, _CHANNELS[color]), dtype=np.uint32)
        for interlace in (False, True):
            blob = _encode(samples, 8, color, interlace=interlace, seed=3)
            ref = np.asarray(PIL.open(io.BytesIO(blob)).convert(mode)).reshape(21, 37, -1)
            assert np.array_equal(ref, samples.astype(np.uint8))           # the encoder of this file is sound
            assert np.array_equal(_decode(blob)["image"].numpy(), ref)
    # and a file that Pillow wrote (its own filter heuristics and compression settings)
    img = rng.integers(0, 256, size=(40, 50, 3), dtype=np.uint8)
    buf = io.BytesIO()
    PIL.fromarray(img).save(buf, format="PNG", optimize=True)
    assert np.array_equal(_decode(buf.getvalue())["image"].numpy(), img)


@pytest.mark.parametrize("depth", [1, 2, 4, 8])
def test_palette_images(depth: int) -> None:
    rng = np.random.default_rng(depth)
    size = 2 ** depth
    palette = rng.integers(0, 256, size=(size, 3), dtype=np.uint8)
    idx = rng.integers(0, size, size=(13, 19, 1), dtype=np.uint32)
    for interlace in (False, True):
        out = _decode(_encode(idx, depth, 3, interlace=interlace, palette=palette))
        assert out["channels"] == 3 and np.array_equal(out["image"].numpy(), palette[idx[..., 0]])
        trns = bytes(rng.integers(0, 256, size=max(1, size // 2), dtype=np.uint8))
        out = _decode(_encode(idx, depth, 3, interlace=interlace, palette=palette, trns=trns))
        alpha = np.array(list(trns) + [255] * (size - len(trns)), dtype=np.uint8)
        want = np.concatenate([palette[idx[..., 0]], alpha[idx[..., 0]][..., None]], -1)
        assert out["channels"] == 4 and np.array_equal(out["image"].numpy(), want)
    short = palette[: max(1, size // 2)]
    bad = np.full((2, 2, 1), size - 1, dtype=np.uint32)
    if size > 1 and len(short) < size:
        with pytest.raises(ValueError, match="palette index"):
            _decode(_encode(bad, depth, 3, palette=short))


def test_damaged_files_are_refused() -> None:
    good = _encode(np.zeros((4, 4, 3), dtype=np.uint32), 8, 2)
    flipped = bytearray(good)
    flipped[good.index(b"IDAT") + 6] ^= 0x40
    with pytest.raises(ValueError, match="checksum"):
        _decode(bytes(flipped))
    with pytest.raises(ValueError, match="truncated"):
        _decode(good[:-14])
    with pytest.raises(ValueError):
        _decode(good[:8] + _chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 4, 3, 2, 0, 0, 0)) + good[33:])   # depth 3
    with pytest.raises(ValueError):
        _decode(good[:8] + _chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 4, 16, 3, 0, 0, 0)) + good[33:])  # palette, 16 bit
    with pytest.raises(ValueError, match="inflated"):
        _decode(good[:8] + _chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 5, 8, 2, 0, 0, 0)) + good[33:])   # one row short
    with pytest.raises(ValueError):
        _decode(b"GIF89a" + b"\x00" * 32)
