"""Per-operator tests of the native data pipeline: outputs over two epochs with
``reset()``, ``state_dict()``/``load_state_dict()`` round trips and error
propagation (modelled on the reference's tests/unit/data/data_pipeline/*)."""
from __future__ import annotations

import io
import struct
import zipfile
from pathlib import Path

import pytest
import torch

from fairseq2_b200.data import (Collater, DataPipeline, DataPipelineError, FileMapper, create_bucket_sizes, list_files,
                                read_iterator, read_sequence, read_zipped_records)
from fairseq2_b200.data.audio import AudioDecoder, WaveformToFbankConverter
from fairseq2_b200.data.text import StrSplitter, StrToIntConverter, StrToTensorConverter, read_text


def _two_epochs(p):
    a = list(p)
    p.reset()
    b = list(p)
    return a, b


def test_read_sequence_and_reset() -> None:
    p = read_sequence([1, 2, 3, 4]).and_return()
    a, b = _two_epochs(p)
    assert a == b == [1, 2, 3, 4]


def test_state_dict_roundtrip_mid_epoch() -> None:
    p = read_sequence(list(range(10))).map(lambda x: x * 2).and_return()
    it = iter(p)
    assert [next(it) for _ in range(4)] == [0, 2, 4, 6]
    sd = p.state_dict()
    assert [next(it) for _ in range(2)] == [8, 10]
    p.load_state_dict(sd)
    assert list(p) == [8, 10, 12, 14, 16, 18]


def test_map_selector_and_parallel() -> None:
    data = [{"a": {"b": i}, "c": [i, i + 1]} for i in range(8)]
    p = read_sequence(data).map(lambda x: x + 100, selector="a.b,c[1]", num_parallel_calls=4).and_return()
    out = list(p)
    assert [o["a"]["b"] for o in out] == [100 + i for i in range(8)]
    assert [o["c"] for o in out] == [[i, i + 101] for i in range(8)]
    assert data[0]["a"]["b"] == 0  # inputs are not mutated


def test_map_error_breaks_pipeline() -> None:
    def boom(x):
        if x == 2:
            raise ValueError("bad example")
        return x

    p = read_sequence([1, 2, 3]).map(boom).and_return()
    it = iter(p)
    assert next(it) == 1
    with pytest.raises(ValueError, match="bad example"):
        next(it)
    assert p.is_broken
    with pytest.raises(DataPipelineError):
        next(iter(p))


def test_filter_skip_take_repeat() -> None:
    p = read_sequence(list(range(10))).filter(lambda x: x % 2 == 0).skip(1).take(3).and_return()
    assert list(p) == [2, 4, 6]
    p = read_sequence([1, 2]).repeat(3).and_return()
    assert list(p) == [1, 2, 1, 2, 1, 2]
    p = read_sequence([]).repeat().and_return()
    assert list(p) == []


def test_bucket_and_shard() -> None:
    p = read_sequence(list(range(7))).bucket(3).and_return()
    assert list(p) == [[0, 1, 2], [3, 4, 5], [6]]
    p = read_sequence(list(range(7))).bucket(3, drop_remainder=True).and_return()
    assert list(p) == [[0, 1, 2], [3, 4, 5]]
    assert list(read_sequence(list(range(7))).shard(1, 3).and_return()) == [1, 4]
    assert list(read_sequence(list(range(7))).shard(0, 3, allow_uneven=True).and_return()) == [0, 3, 6]
    with pytest.raises(ValueError):
        read_sequence([1]).shard(3, 3)


def test_bucket_by_length() -> None:
    seqs = [torch.arange(n) for n in (1, 5, 2, 6, 2, 4, 1)]
    p = read_sequence(seqs).bucket_by_length([(3, 2), (2, 6)]).and_return()
    out = [[len(t) for t in b] for b in p]
    assert out == [[5, 6], [1, 2, 2], [4, 1]]
    with pytest.raises(DataPipelineError):
        list(read_sequence([torch.arange(9)]).bucket_by_length([(1, 4)]).and_return())
    assert list(read_sequence([torch.arange(9)]).bucket_by_length([(1, 4)], skip_above_max_examples=True).and_return()) == []


def test_dynamic_bucket() -> None:
    p = read_sequence([1, 2, 3, 4, 5, 6]).dynamic_bucket(5, lambda x: x).and_return()
    assert list(p) == [[1, 2, 3], [4, 5], [6]]
    p = read_sequence([1, 2, 3, 4, 5, 6]).dynamic_bucket(100, lambda x: x, max_num_examples=4).and_return()
    assert list(p) == [[1, 2, 3, 4], [5, 6]]


def test_shuffle_is_seeded_permutation_and_resumable() -> None:
    p = read_sequence(list(range(50))).shuffle(16, seed=3).and_return()
    a = list(p)
    assert sorted(a) == list(range(50)) and a != list(range(50))
    p.reset(reset_rng=True)
    assert list(p) == a
    p.reset(reset_rng=True)
    it = iter(p)
    head = [next(it) for _ in range(20)]
    sd = p.state_dict()
    tail = list(it)
    p.load_state_dict(sd)
    assert list(p) == tail and head + tail == a


def test_concat_zip_round_robin_sample() -> None:
    a = read_sequence([1, 2, 3]).and_return()
    b = read_sequence([10, 20]).and_return()
    assert list(DataPipeline.concat([a, b]).and_return()) == [1, 2, 3, 10, 20]
    a, b = read_sequence([1, 2, 3]).and_return(), read_sequence([10, 20, 30]).and_return()
    assert list(DataPipeline.zip([a, b], names=["x", "y"]).and_return()) == [{"x": 1, "y": 10}, {"x": 2, "y": 20}, {"x": 3, "y": 30}]
    a, b = read_sequence([1, 2, 3]).and_return(), read_sequence([10, 20]).and_return()
    with pytest.raises(DataPipelineError):
        list(DataPipeline.zip([a, b]).and_return())
    a, b = read_sequence([1, 2, 3]).and_return(), read_sequence([10, 20]).and_return()
    assert list(DataPipeline.zip([a, b], zip_to_shortest=True).and_return()) == [[1, 10], [2, 20]]
    a, b = read_sequence([1, 2, 3, 4]).and_return(), read_sequence([10, 20]).and_return()
    rr = list(DataPipeline.round_robin([a, b]).and_return())
    assert rr == [1, 10, 2, 20, 3, 10, 4, 20]
    a, b = read_sequence([1, 2, 3, 4]).and_return(), read_sequence([10, 20]).and_return()
    assert list(DataPipeline.round_robin([a, b], stop_at_shortest=True).and_return()) == [1, 10, 2, 20]
    a, b = read_sequence(list(range(100))).and_return(), read_sequence(list(range(1000, 1100))).and_return()
    s = list(DataPipeline.sample([a, b], weights=[0.8, 0.2], seed=1).and_return())
    assert {x for x in s if x < 1000} == set(range(100)) and {x for x in s if x >= 1000} == set(range(1000, 1100))


def test_count_constant_yield_from() -> None:
    assert list(DataPipeline.count(5, step=2).take(3).and_return()) == [5, 7, 9]
    assert list(DataPipeline.count(0, key="i").take(2).and_return()) == [{"i": 0}, {"i": 1}]
    assert list(DataPipeline.constant(7).take(2).and_return()) == [7, 7]
    p = read_sequence([1, 2, 3]).yield_from(lambda n: read_sequence(list(range(n))).and_return()).and_return()
    assert list(p) == [0, 0, 1, 0, 1, 2]


def test_prefetch_preserves_order_and_errors() -> None:
    p = read_sequence(list(range(100))).map(lambda x: x + 1).prefetch(8).and_return()
    a, b = _two_epochs(p)
    assert a == b == list(range(1, 101))

    def boom(x):
        if x == 5:
            raise RuntimeError("prefetch failure")
        return x

    p = read_sequence(list(range(10))).map(boom).prefetch(2).and_return()
    with pytest.raises(RuntimeError, match="prefetch failure"):
        list(p)


def test_pack() -> None:
    seqs = [torch.full((n,), i + 1) for i, n in enumerate((3, 4, 2, 5))]
    p = read_sequence(seqs).pack(num_elements=8, max_seq_len=8, pad_value=0, truncate=False).and_return()
    out = list(p)                                           # whole sequences only; the last buffer is kept
    assert out[0]["seqs"].tolist() == [1, 1, 1, 2, 2, 2, 2, 0] and out[0]["seq_lens"] == [3, 4]
    assert out[1]["seqs"].tolist() == [3, 3, 4, 4, 4, 4, 4, 0] and out[1]["seq_lens"] == [2, 5]
    p = read_sequence(seqs).pack(num_elements=8, max_seq_len=8, drop_remainder=False).and_return()   # truncating
    out = list(p)
    assert out[0]["seqs"].tolist() == [1, 1, 1, 2, 2, 2, 2, 3] and out[0]["seq_lens"] == [3, 4, 1]
    # the next buffer starts again with the last token that went in
    assert out[1]["seqs"].tolist() == [3, 3, 4, 4, 4, 4, 4, 0] and out[1]["seq_lens"] == [2, 5]
    # pieces are at most `max_seq_len` long; the rest of a sequence follows as its own piece
    p = read_sequence([torch.arange(1, 8)]).pack(num_elements=8, max_seq_len=3, drop_remainder=False).and_return()
    out = list(p)
    assert out[0]["seqs"].tolist() == [1, 2, 3, 4, 5, 6, 7, 0] and out[0]["seq_lens"] == [3, 3, 1]
    with pytest.raises(DataPipelineError, match="too long to pack"):
        list(read_sequence([torch.arange(9)]).pack(num_elements=8, max_seq_len=8, truncate=False).and_return())


def test_collater_pads_and_stacks() -> None:
    bucket = [{"ids": torch.tensor([1, 2, 3]), "feat": torch.ones(2), "name": "a"},
              {"ids": torch.tensor([4]), "feat": torch.zeros(2), "name": "b"}]
    with pytest.raises(ValueError):
        Collater()(bucket)
    out = Collater(pad_value=0)(bucket)
    assert out["ids"]["seqs"].tolist() == [[1, 2, 3], [4, 0, 0]]
    assert out["ids"]["seq_lens"] == [3, 1] and out["ids"]["is_ragged"] is True
    assert out["name"] == ["a", "b"]
    out = Collater(pad_value=0, pad_to_multiple=4)(bucket)
    assert out["ids"]["seqs"].shape == (2, 4)
    p = read_sequence(bucket).bucket(2).collate(pad_value=-1).and_return()
    assert next(iter(p))["ids"]["seqs"].tolist() == [[1, 2, 3], [4, -1, -1]]


def test_text_reader_and_converters(tmp_path: Path) -> None:
    f = tmp_path / "a.tsv"
    f.write_text("1\t10 20\thello\r\n\n2\t30 40\tworld\n")
    lines = list(read_text(f, rtrim=True, skip_empty=True).and_return())
    assert lines == ["1\t10 20\thello", "2\t30 40\tworld"]
    p = (read_text(f, rtrim=True, skip_empty=True).map(StrSplitter(names=["id", "nums", "txt"]))
         .map(StrToIntConverter(), selector="id").map(StrToTensorConverter(dtype=torch.int64), selector="nums").and_return())
    out = list(p)
    assert out[0]["id"] == 1 and out[1]["nums"].tolist() == [30, 40] and out[1]["txt"] == "world"
    assert StrSplitter(sep=",", indices=[1])("a,b,c") == ["b"]
    with pytest.raises(ValueError):
        StrToIntConverter()("x1")


def test_list_files_file_mapper_and_zip(tmp_path: Path) -> None:
    for n in ("f10.txt", "f2.txt", "g1.bin"):
        (tmp_path / n).write_bytes(n.encode())
    files = list(list_files(tmp_path, pattern="*.txt").and_return())
    assert [Path(f).name for f in files] == ["f2.txt", "f10.txt"]  # natural order
    m = FileMapper(root_dir=tmp_path)
    out = m("f2.txt")
    assert bytes(out["data"]) == b"f2.txt"
    assert bytes(m("f10.txt:1:3")["data"]) == b"10."
    z = tmp_path / "a.zip"
    with zipfile.ZipFile(z, "w", zipfile.ZIP_DEFLATED) as zf:
        zf.writestr("x.txt", "hello " * 100)
        zf.writestr("y.txt", "bye")
    recs = [bytes(r) for r in read_zipped_records(z).and_return()]
    assert recs == [b"hello " * 100, b"bye"]


class _CountingIterator:
    """Module-level so that it can be pickled into the pipeline state."""

    def __init__(self) -> None:
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        if self.i >= 5:
            raise StopIteration
        self.i += 1
        return self.i


def _reset_counting(it):
    it.i = 0
    return it


def test_read_iterator_state() -> None:
    It, reset = _CountingIterator, _reset_counting
    p = read_iterator(It(), reset_fn=reset, infinite=False).and_return()
    it = iter(p)
    assert [next(it), next(it)] == [1, 2]
    sd = p.state_dict()
    assert list(it) == [3, 4, 5]
    p.load_state_dict(sd)
    assert list(p) == [3, 4, 5]
    p.reset()
    assert list(p) == [1, 2, 3, 4, 5]


def test_audio_decode_and_fbank() -> None:
    sr, n = 16000, 16000
    t = torch.arange(n) / sr
    wav = (0.5 * torch.sin(2 * torch.pi * 440 * t) * 32767).to(torch.int16)
    buf = io.BytesIO()
    data = wav.numpy().tobytes()
    buf.write(b"RIFF" + struct.pack("<I", 36 + len(data)) + b"WAVE")
    buf.write(b"fmt " + struct.pack("<IHHIIHH", 16, 1, 1, sr, sr * 2, 2, 16))
    buf.write(b"data" + struct.pack("<I", len(data)) + data)
    from fairseq2_b200.data import MemoryBlock

    out = AudioDecoder(dtype=torch.float32)(MemoryBlock(buf.getvalue()))
    assert out["sample_rate"] == 16000.0 and out["waveform"].shape == (n,)
    assert torch.allclose(out["waveform"], wav.float() / 32768, atol=1e-6)
    fb = WaveformToFbankConverter(num_mel_bins=80, waveform_scale=2 ** 15)({"waveform": out["waveform"], "sample_rate": 16000.0})
    assert fb["fbank"].shape == (98, 80) and torch.isfinite(fb["fbank"]).all()
    peak_bin = int(fb["fbank"].mean(0).argmax())
    assert 10 <= peak_bin <= 25  # 440 Hz lands in the low mel bins


def test_create_bucket_sizes() -> None:
    sizes = create_bucket_sizes(max_num_elements=16, max_seq_len=8, min_seq_len=2)
    assert sizes[-1] == (2, 8) and all(b * s <= 16 for b, s in sizes)
    assert [s for _, s in sizes] == sorted(s for _, s in sizes)


def test_image_decoder_jpeg_matches_libjpeg() -> None:
    """Baseline JPEG (grayscale, 4:4:4, 4:2:2, 4:2:0, restart markers) decoded by the native runtime vs Pillow."""
    import io

    import numpy as np

    PIL = pytest.importorskip("PIL.Image")
    from fairseq2_b200.data.data_pipeline import MemoryBlock
    from fairseq2_b200.data.image import ImageDecoder

    y, x = np.mgrid[0:67, 0:93]
    rgb = np.stack([(x * 2 + y) % 256, (x + y * 3) % 256, (x * y // 7) % 256], -1).astype(np.uint8)
    rgb = (0.5 * rgb + 0.5 * np.roll(rgb, 3, 0)).astype(np.uint8)
    dec = ImageDecoder()
    cases = [("RGB", {"subsampling": 0}), ("RGB", {"subsampling": 1}), ("RGB", {"subsampling": 2}), ("L", {}),
             ("RGB", {"subsampling": 2, "restart_marker_rows": 1})]
    for mode, kw in cases:
        im = PIL.fromarray(rgb if mode == "RGB" else rgb[..., 0])
        buf = io.BytesIO()
        im.save(buf, format="JPEG", quality=90, **kw)
        data = buf.getvalue()
        out = dec(MemoryBlock(data))
        ref = np.asarray(PIL.open(io.BytesIO(data)).convert(mode))
        ref = ref if ref.ndim == 3 else ref[..., None]
        got = out["image"].numpy()
        assert got.shape == ref.shape and out["bit_depth"] == 8.0
        assert np.abs(got.astype(int) - ref.astype(int)).max() <= 4, (mode, kw)
    with pytest.raises(Exception):
        dec(MemoryBlock(b"\xff\xd8\xff\xc2\x00\x0b\x08\x00\x10\x00\x10\x01\x01\x11\x00"))      # no scan


def test_image_decoder_progressive_jpeg_matches_libjpeg() -> None:
    """Progressive JPEG (DC/AC first and refinement scans, non-interleaved AC scans, optimised tables, restart
    intervals) vs Pillow; the same pixels through the sequential and the progressive path agree exactly because
    both reconstruct the same coefficients."""
    import io

    import numpy as np

    PIL = pytest.importorskip("PIL.Image")
    from fairseq2_b200.data.data_pipeline import MemoryBlock
    from fairseq2_b200.data.image import ImageDecoder

    rng = np.random.default_rng(0)
    y, x = np.mgrid[0:131, 0:157]
    rgb = np.stack([(x * 2 + y) % 256, (x + y * 3) % 256, (x * y // 7) % 256], -1).astype(np.float64)
    rgb = np.clip(0.6 * rgb + 0.4 * np.roll(rgb, 5, 1) + rng.normal(0, 6, rgb.shape), 0, 255).astype(np.uint8)
    dec = ImageDecoder()
    cases = [("RGB", 0, 90, {}), ("RGB", 1, 75, {}), ("RGB", 2, 95, {}), ("L", 0, 85, {}),
             ("RGB", 2, 60, {"restart_marker_blocks": 3}), ("L", 0, 98, {"restart_marker_rows": 2})]
    for mode, sub, quality, extra in cases:
        im = PIL.fromarray(rgb if mode == "RGB" else rgb[..., 1])
        kw = {"subsampling": sub} if mode == "RGB" else {}
        prog, seq = io.BytesIO(), io.BytesIO()
        im.save(prog, format="JPEG", quality=quality, progressive=True, **kw, **extra)
        im.save(seq, format="JPEG", quality=quality, progressive=False, **kw)
        assert b"\xff\xc2" in prog.getvalue()
        got = dec(MemoryBlock(prog.getvalue()))["image"].numpy()
        ref = np.asarray(PIL.open(io.BytesIO(prog.getvalue())).convert(mode))
        ref = ref if ref.ndim == 3 else ref[..., None]
        assert got.shape == ref.shape
        assert np.abs(got.astype(int) - ref.astype(int)).max() <= 4, (mode, sub, quality)
        same = dec(MemoryBlock(seq.getvalue()))["image"].numpy()
        assert np.array_equal(got, same), (mode, sub, quality)


def test_read_text_reencodes_with_iconv(tmp_path) -> None:
    from fairseq2_b200.data.text import read_text

    p = tmp_path / "latin1.txt"
    p.write_bytes("señor\nmañana\n".encode("latin-1"))
    assert list(read_text(p, encoding="latin1", rtrim=True).and_return()) == ["señor", "mañana"]
    q = tmp_path / "sjis.txt"
    q.write_bytes("日本語\nテキスト".encode("shift_jis"))
    assert list(read_text(q, encoding="SHIFT_JIS").and_return()) == ["日本語", "テキスト"]
    with pytest.raises(ValueError):
        list(read_text(p, encoding="klingon").and_return())
    with pytest.raises(Exception, match="not valid"):
        list(read_text(q, encoding="utf-16").and_return())  # 15 bytes: a truncated code unit


def test_image_decoder_jpeg_colour_spaces() -> None:
    """Four-component files (CMYK as stored; YCCK converted to CMYK) and three-component files stored without a
    colour transform, against Pillow. Pillow inverts Adobe ink values when it loads a file; the decoder passes
    them on with the polarity of the file, as libjpeg does."""
    import io

    import numpy as np

    PIL = pytest.importorskip("PIL.Image")
    from fairseq2_b200.data.data_pipeline import MemoryBlock
    from fairseq2_b200.data.image import ImageDecoder

    y, x = np.mgrid[0:67, 0:93]
    rgb = np.stack([(x * 2 + y) % 256, (x + y * 3) % 256, (x * y // 7) % 256], -1).astype(np.uint8)
    rgb = (0.5 * rgb + 0.5 * np.roll(rgb, 3, 0)).astype(np.uint8)
    cmyk = np.concatenate([rgb, ((x + 2 * y) % 256).astype(np.uint8)[..., None]], -1)
    dec = ImageDecoder()
    for progressive in (False, True):
        buf = io.BytesIO()
        PIL.fromarray(cmyk, mode="CMYK").save(buf, format="JPEG", quality=92, progressive=progressive)
        data = buf.getvalue()
        out = dec(MemoryBlock(data))
        ref = 255 - np.asarray(PIL.open(io.BytesIO(data))).astype(int)
        assert out["channels"] == 4 and out["image"].shape == (67, 93, 4)
        assert np.abs(out["image"].numpy().astype(int) - ref).max() <= 2
        # the same scan data declared as YCCK: byte 11 of the Adobe segment is the transform flag
        at = data.index(b"Adobe")
        assert data[at + 11] == 0
        ycck = data[: at + 11] + b"\x02" + data[at + 12:]
        out = dec(MemoryBlock(ycck))
        ref = 255 - np.asarray(PIL.open(io.BytesIO(ycck))).astype(int)
        assert np.abs(out["image"].numpy().astype(int) - ref).max() <= 4
    buf = io.BytesIO()
    PIL.fromarray(rgb).save(buf, format="JPEG", quality=92, keep_rgb=True)       # RGB planes, no YCbCr transform
    out = dec(MemoryBlock(buf.getvalue()))
    ref = np.asarray(PIL.open(io.BytesIO(buf.getvalue())).convert("RGB")).astype(int)
    assert out["channels"] == 3 and np.abs(out["image"].numpy().astype(int) - ref).max() <= 2
