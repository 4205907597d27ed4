"""FLAC decoding of the native audio decoder against streams produced by a small bit-exact FLAC writer kept in this
file (no FLAC library is available to the test environment): every subframe type, Rice and escaped partitions,
wasted bits, the four channel assignments, explicit and coded block sizes, and corruption detection through the
frame CRCs."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from fairseq2_b200.data import MemoryBlock
from fairseq2_b200.data.audio import AudioDecoder


class _Bits:
    def __init__(self) -> None:
        self.acc, self.n, self.out = 0, 0, bytearray()

    def put(self, value: int, nbits: int) -> None:
        if nbits == 0:
            return
        value &= (1 << nbits) - 1
        self.acc = (self.acc << nbits) | value
        self.n += nbits
        while self.n >= 8:
            self.n -= 8
            self.out.append((self.acc >> self.n) & 0xFF)
        self.acc &= (1 << self.n) - 1

    def unary(self, zeros: int) -> None:
        while zeros >= 32:
            self.put(0, 32)
            zeros -= 32
        self.put(1, zeros + 1)

    def align(self) -> None:
        if self.n:
            self.put(0, 8 - self.n)


def _crc(data: bytes, poly: int, width: int) -> int:
    c, top, mask = 0, 1 << (width - 1), (1 << width) - 1
    for b in data:
        c ^= b << (width - 8)
        for _ in range(8):
            c = ((c << 1) ^ poly) & mask if c & top else (c << 1) & mask
    return c


def _utf8(n: int) -> bytes:
    if n < 0x80:
        return bytes([n])
    out, lead_bits = [], 6
    while n >= (1 << lead_bits):
        out.append(0x80 | (n & 0x3F))
        n >>= 6
        lead_bits -= 1
    lead = (0xFF << (lead_bits + 1)) & 0xFF
    return bytes([lead | n] + out[::-1])


def _rice(w: _Bits, residual: list[int], order: int, block: int, porder: int, escape_first: bool, rice2: bool) -> None:
    w.put(1 if rice2 else 0, 2)
    w.put(porder, 4)
    pbits = 5 if rice2 else 4
    parts = 1 << porder
    i = 0
    for part in range(parts):
        count = (block >> porder) - (order if part == 0 else 0)
        chunk = residual[i:i + count]
        i += count
        if escape_first and part == 0:
            w.put((1 << pbits) - 1, pbits)
            raw = max([1] + [abs(v).bit_length() + 1 for v in chunk])
            w.put(raw, 5)
            for v in chunk:
                w.put(v, raw)
            continue
        mean = sum(abs(v) for v in chunk) / max(1, len(chunk))
        k = min(max(int(mean).bit_length(), 0), (1 << pbits) - 2)
        w.put(k, pbits)
        for v in chunk:
            u = (v << 1) if v >= 0 else ((-v << 1) - 1)
            w.unary(u >> k)
            w.put(u & ((1 << k) - 1), k)


def _subframe(w: _Bits, s: list[int], bps: int, kind: tuple) -> None:
    block = len(s)
    wasted = 0
    if kind[0] != "constant" and any(s) and kind[-1] == "wasted":
        while all(v % (1 << (wasted + 1)) == 0 for v in s):
            wasted += 1
        kind = kind[:-1]
    elif kind[-1] == "wasted":
        kind = kind[:-1]
    s = [v >> wasted for v in s]
    bps -= wasted
    code = {"constant": 0, "verbatim": 1}.get(kind[0])
    if kind[0] == "fixed":
        code = 8 + kind[1]
    if kind[0] == "lpc":
        code = 31 + len(kind[1])
    w.put(0, 1)
    w.put(code, 6)
    if wasted:
        w.put(1, 1)
        w.unary(wasted - 1)
    else:
        w.put(0, 1)
    if kind[0] == "constant":
        w.put(s[0], bps)
    elif kind[0] == "verbatim":
        for v in s:
            w.put(v, bps)
    elif kind[0] == "fixed":
        order = kind[1]
        coefs = {0: [], 1: [1], 2: [2, -1], 3: [3, -3, 1], 4: [4, -6, 4, -1]}[order]
        for v in s[:order]:
            w.put(v, bps)
        res = [s[i] - sum(c * s[i - 1 - j] for j, c in enumerate(coefs)) for i in range(order, block)]
        _rice(w, res, order, block, kind[2], kind[3], kind[4])
    else:
        coefs, precision, shift = kind[1], kind[2], kind[3]
        order = len(coefs)
        for v in s[:order]:
            w.put(v, bps)
        w.put(precision - 1, 4)
        w.put(shift, 5)
        for c in coefs:
            w.put(c, precision)
        res = [s[i] - (sum(c * s[i - 1 - j] for j, c in enumerate(coefs)) >> shift) for i in range(order, block)]
        _rice(w, res, order, block, kind[4], False, kind[5])


_BS_CODES = {192: 1, 576: 2, 1152: 3, 2304: 4, 4608: 5, 256: 8, 512: 9, 1024: 10, 2048: 11, 4096: 12}
_SS_CODES = {8: 1, 12: 2, 16: 4, 20: 5, 24: 6, 32: 7}


def write_flac(pcm: np.ndarray, bps: int, rate: int, plan: list[dict]) -> bytes:
    """``pcm``: int64 [frames, channels]; ``plan``: per frame ``{"block", "assign", "kinds"}``."""
    frames, ch = pcm.shape
    out = bytearray(b"fLaC")
    max_block = max(f["block"] for f in plan)
    info = _Bits()
    info.put(min(f["block"] for f in plan[:-1] or plan), 16)
    info.put(max_block, 16)
    info.put(0, 24)
    info.put(0, 24)
    info.put(rate, 20)
    info.put(ch - 1, 3)
    info.put(bps - 1, 5)
    info.put(frames, 36)
    info.put(0, 128)
    out += bytes([0x00, 0, 0, 34]) + bytes(info.out)           # STREAMINFO, not last
    out += bytes([0x84, 0, 0, 8]) + b"\x04\x00\x00\x00abcd"    # VORBIS_COMMENT-typed block (skipped), last
    pos = 0
    for nr, f in enumerate(plan):
        block, assign = f["block"], f["assign"]
        x = pcm[pos:pos + block]
        pos += block
        w = _Bits()
        w.put(0b111111111111100, 15)
        w.put(0, 1)
        bs_code = _BS_CODES.get(block, 6 if block <= 256 else 7) if f.get("coded_bs", True) else (6 if block <= 256 else 7)
        w.put(bs_code, 4)
        sr_code = f.get("sr_code", 0)
        w.put(sr_code, 4)
        w.put({"independent": ch - 1, "left_side": 8, "right_side": 9, "mid_side": 10}[assign], 4)
        w.put(_SS_CODES[bps] if f.get("explicit_ss", False) else 0, 3)
        w.put(0, 1)
        for b in _utf8(nr):
            w.put(b, 8)
        if bs_code == 6:
            w.put(block - 1, 8)
        elif bs_code == 7:
            w.put(block - 1, 16)
        if sr_code == 12:
            w.put(rate // 1000, 8)
        elif sr_code == 13:
            w.put(rate, 16)
        elif sr_code == 14:
            w.put(rate // 10, 16)
        w.put(_crc(bytes(w.out), 0x07, 8), 8)
        chans = [[int(v) for v in x[:, c]] for c in range(ch)]
        widths = [bps] * ch
        if assign == "left_side":
            chans = [chans[0], [a - b for a, b in zip(chans[0], chans[1])]]
            widths = [bps, bps + 1]
        elif assign == "right_side":
            chans = [[a - b for a, b in zip(chans[0], chans[1])], chans[1]]
            widths = [bps + 1, bps]
        elif assign == "mid_side":
            chans = [[(a + b) >> 1 for a, b in zip(chans[0], chans[1])], [a - b for a, b in zip(chans[0], chans[1])]]
            widths = [bps, bps + 1]
        for c in range(ch):
            _subframe(w, chans[c], widths[c], f["kinds"][c])
        w.align()
        body = bytes(w.out)
        out += body + _crc(body, 0x8005, 16).to_bytes(2, "big")
    assert pos == frames
    return bytes(out)


def _signal(frames: int, ch: int, bps: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    t = np.arange(frames)[:, None]
    amp = (1 << (bps - 1)) * 0.4
    x = amp * np.sin(2 * np.pi * t * (0.01 + 0.003 * np.arange(ch))) + rng.normal(0, amp * 0.01, (frames, ch))
    return np.clip(np.round(x), -(1 << (bps - 1)), (1 << (bps - 1)) - 1).astype(np.int64)


def _decode(data: bytes, **kw):  # type: ignore[no-untyped-def]
    return AudioDecoder(**kw)(MemoryBlock(data))


def test_flac_mono_all_subframe_types() -> None:
    pcm = _signal(4096 + 1000 + 192 + 37, 1, 16, 0)
    pcm[4096:5096] = 1234                                    # a constant block
    pcm[5096:5288] &= ~7                                     # three wasted bits
    plan = [
        {"block": 4096, "assign": "independent", "kinds": [("lpc", [1900, -900], 12, 10, 2, False)]},
        {"block": 1000, "assign": "independent", "kinds": [("constant",)], "sr_code": 13},
        {"block": 192, "assign": "independent", "kinds": [("fixed", 2, 0, False, False, "wasted")], "explicit_ss": True},
        {"block": 37, "assign": "independent", "kinds": [("verbatim",)], "sr_code": 5},
    ]
    out = _decode(write_flac(pcm, 16, 16000, plan))
    assert out["sample_rate"] == 16000.0 and out["format"] == "FLAC/PCM_16"
    assert out["waveform"].dtype == torch.int16 and out["waveform"].shape == (pcm.shape[0],)
    assert torch.equal(out["waveform"].long(), torch.from_numpy(pcm[:, 0]))
    f = _decode(write_flac(pcm, 16, 16000, plan), dtype=torch.float32, keepdim=True)["waveform"]
    assert f.shape == (pcm.shape[0], 1)
    torch.testing.assert_close(f[:, 0], torch.from_numpy(pcm[:, 0] / 32768.0).float())


@pytest.mark.parametrize("assign", ["independent", "left_side", "right_side", "mid_side"])
@pytest.mark.parametrize("bps", [16, 24])
def test_flac_stereo_channel_assignments(assign: str, bps: int) -> None:
    pcm = _signal(2 * 1152 + 500, 2, bps, 3)
    pcm[:, 1] = pcm[:, 0] // 2 + _signal(pcm.shape[0], 1, bps - 4, 9)[:, 0]     # correlated channels, odd sums
    kinds = [("fixed", 3, 2, True, False), ("fixed", 1, 0, False, True)]
    plan = [{"block": 1152, "assign": assign, "kinds": kinds},
            {"block": 1152, "assign": assign, "kinds": [("fixed", 4, 3, False, False), ("fixed", 0, 1, False, False)]},
            {"block": 500, "assign": assign, "kinds": kinds[::-1], "coded_bs": False}]
    out = _decode(write_flac(pcm, bps, 44100, plan))
    assert out["format"] == f"FLAC/PCM_{bps}" and out["sample_rate"] == 44100.0
    assert out["waveform"].dtype == (torch.int16 if bps == 16 else torch.int32)
    assert torch.equal(out["waveform"].long(), torch.from_numpy(pcm))


def test_flac_many_frames_and_32_bit() -> None:
    pcm = _signal(200 * 256, 1, 32, 5)
    plan = [{"block": 256, "assign": "independent", "kinds": [("fixed", 2, 1, False, True)]} for _ in range(200)]
    out = _decode(write_flac(pcm, 32, 48000, plan))        # frame numbers above 127 use two-byte codes
    assert torch.equal(out["waveform"].long(), torch.from_numpy(pcm[:, 0]))


def test_flac_corruption_is_detected() -> None:
    pcm = _signal(1024, 1, 16, 1)
    data = bytearray(write_flac(pcm, 16, 16000, [{"block": 1024, "assign": "independent",
                                                   "kinds": [("fixed", 2, 0, False, False)]}]))
    bad = bytearray(data)
    bad[len(bad) // 2] ^= 0x10
    with pytest.raises(ValueError, match="FLAC"):
        _decode(bytes(bad))
    with pytest.raises(ValueError, match="FLAC"):
        _decode(bytes(data[:-40]))
    hdr = bytearray(data)
    hdr[4 + 4 + 34 + 4 + 8 + 2] ^= 0x01                       # inside the frame header: CRC-8 catches it
    with pytest.raises(ValueError, match="FLAC"):
        _decode(bytes(hdr))
    with pytest.raises(ValueError, match="Ogg"):
        _decode(b"OggS" + bytes(60))
