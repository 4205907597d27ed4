"""The native SentencePiece runtime against the ``sentencepiece`` package: models are trained here with the package,
then every segmentation, id and decoded string of the native runtime must equal the package's."""
from __future__ import annotations

import io
import pickle
import random
from collections import Counter

import pytest
import torch

spm = pytest.importorskip("sentencepiece")

from fairseq2_b200.data.data_pipeline import read_sequence  # noqa: E402
from fairseq2_b200.data.tokenizers.sentencepiece import (SentencePieceDecoder, SentencePieceEncoder,  # noqa: E402
                                                         SentencePieceModel)

_WORDS = ["hello", "world", "token", "izer", "native", "b200", "über", "naïve", "日本語", "テスト", "café", "running",
          "runner", "runs", "12345", "3.14", "foo_bar", "Hello", "WORLD", "ﬁne", "①", "ｆｕｌｌ", "the", "a", "of", "and",
          "to", "in", "is", "that", "it", "for", "tokenization", "segment", "piece", "sentence", "model", "unigram", "bpe"]

_PROBES = ["hello  world <sep> naïve ｆｕｌｌ xyz\t日本", "", "   ", " a ", "hello", "Hello WORLD 12345 3.14", "zzz qqq",
           "①②③ ﬁne ﬁﬁ", "tokenization of the sentence piece model", "<sep><sep> x<sep>", "<ctl> hi <s> </s>",
           "日本語テスト日本", "emoji 😀 here", "á é", "tab\there\nnewline", "ＡＢＣ　ｄｅｆ", "x" * 50, "unigramunigrambpe",
           "  lead and trail  ", "a  b   c"]


def _corpus() -> list[str]:
    rng = random.Random(0)
    return [" ".join(rng.choice(_WORDS) for _ in range(rng.randint(3, 12))) for _ in range(3000)]


_CONFIGS = {
    "unigram": ("unigram", {}),
    "bpe": ("bpe", {}),
    "unigram_byte_fallback": ("unigram", {"byte_fallback": True}),
    "bpe_byte_fallback": ("bpe", {"byte_fallback": True}),
    "char": ("char", {}),
    "word": ("word", {}),
    "unigram_raw_whitespace": ("unigram", {"add_dummy_prefix": False, "remove_extra_whitespaces": False}),
    "bpe_whitespace_suffix": ("bpe", {"treat_whitespace_as_suffix": True}),
    "unigram_identity": ("unigram", {"normalization_rule_name": "identity"}),
    "unigram_case_folding": ("unigram", {"normalization_rule_name": "nmt_nfkc_cf"}),
    "bpe_keep_whitespace": ("bpe", {"remove_extra_whitespaces": False}),
}


@pytest.fixture(scope="module")
def trained(tmp_path_factory: pytest.TempPathFactory) -> dict[str, tuple]:
    d = tmp_path_factory.mktemp("spm_native")
    lines = _corpus()
    out = {}
    for name, (kind, extra) in _CONFIGS.items():
        blob = io.BytesIO()
        spm.SentencePieceTrainer.train(sentence_iterator=iter(lines), model_writer=blob,
                                       vocab_size=40 if kind == "word" else 400, model_type=kind,
                                       user_defined_symbols=["<sep>"], control_symbols=["<ctl>"],
                                       hard_vocab_limit=False, minloglevel=2, **extra)
        path = d / f"{name}.model"
        path.write_bytes(blob.getvalue())
        out[name] = (path, spm.SentencePieceProcessor(model_file=str(path)))
    return out


@pytest.mark.parametrize("name", list(_CONFIGS))
def test_native_runtime_matches_the_package(trained: dict[str, tuple], name: str) -> None:
    path, ref = trained[name]
    model = SentencePieceModel(path)
    assert model.vocabulary_size == ref.GetPieceSize()
    assert (model.unk_idx, model.bos_idx, model.eos_idx, model.pad_idx) == (ref.unk_id(), ref.bos_id(), ref.eos_id(), None)
    for i in range(ref.GetPieceSize()):
        assert model.index_to_token(i) == ref.IdToPiece(i) and model.token_to_index(ref.IdToPiece(i)) == i
    assert model.token_to_index("no such piece") == ref.unk_id()
    for text in _PROBES + _corpus()[:150]:
        ids = ref.EncodeAsIds(text)
        assert model.encode(text) == ids, text
        assert model.encode_as_tokens(text) == ref.EncodeAsPieces(text), text
        assert model.decode(ids) == ref.DecodeIds(ids), text
        assert model.decode_from_tokens(ref.EncodeAsPieces(text)) == ref.DecodePieces(ref.EncodeAsPieces(text)), text


def test_nbest_matches_the_package(trained: dict[str, tuple]) -> None:
    path, ref = trained["unigram"]
    model = SentencePieceModel(path)
    for text in ("tokenization of the sentence", "hello world", "running runner runs"):
        mine = model.nbest_encode(text, 5)
        theirs = ref.NBestEncodeAsIds(text, 5)
        assert mine[0][0] == ref.EncodeAsIds(text)
        scores = [s for _, s in mine]
        assert scores == sorted(scores, reverse=True) and len(mine) == len(theirs)
        # equal-score candidates may come in either order: compare as sets
        assert sorted(map(tuple, (ids for ids, _ in mine))) == sorted(map(tuple, theirs))
    with pytest.raises(ValueError):
        SentencePieceModel(trained["bpe"][0]).nbest_encode("hello", 3)


def test_sampling_draws_valid_segmentations_and_is_seeded(trained: dict[str, tuple]) -> None:
    text = "tokenization of the sentence piece model"
    for name, alpha in (("unigram", 0.02), ("bpe", 0.3)):
        path, ref = trained[name]
        model = SentencePieceModel(path)
        torch.manual_seed(3)
        enc = SentencePieceEncoder(model, enable_sampling=True, alpha=alpha)
        draws = [tuple(enc(text).tolist()) for _ in range(200)]
        assert len(set(draws)) > 5                                   # it does sample
        for ids in set(draws):                                       # every draw spells the same text
            assert ref.DecodeIds(list(ids)) == text
        torch.manual_seed(3)
        again = SentencePieceEncoder(model, enable_sampling=True, alpha=alpha)
        assert [tuple(again(text).tolist()) for _ in range(200)] == draws
    # a sharp distribution concentrates on the best path; n-best sampling stays inside the n best
    path, ref = trained["unigram"]
    model = SentencePieceModel(path)
    sharp = SentencePieceEncoder(model, enable_sampling=True, alpha=50.0)
    best = tuple(ref.EncodeAsIds(text))
    assert Counter(tuple(sharp(text).tolist()) for _ in range(50))[best] >= 45
    top3 = {tuple(ids) for ids, _ in model.nbest_encode(text, 3)}
    among = SentencePieceEncoder(model, enable_sampling=True, nbest_size=3, alpha=0.5)
    assert {tuple(among(text).tolist()) for _ in range(100)} <= top3


def test_encoder_options_and_pipeline_use(trained: dict[str, tuple]) -> None:
    path, ref = trained["bpe"]
    model = SentencePieceModel(path, control_symbols=["<extra>"])
    assert model.vocabulary_size == ref.GetPieceSize() + 1 and model.token_to_index("<extra>") == ref.GetPieceSize()
    enc = SentencePieceEncoder(model, prefix_tokens=["<s>", "<extra>"], suffix_tokens=["</s>"], reverse=True)
    ids = enc("hello world")
    assert ids.dtype == torch.int64 and ids.tolist() == [2, *ref.EncodeAsIds("hello world")[::-1], ref.GetPieceSize(), 1]
    assert enc.encode_as_tokens("hello world") == ["</s>", *ref.EncodeAsPieces("hello world")[::-1], "<extra>", "<s>"]  # reversed as a whole
    dec = SentencePieceDecoder(model, reverse=True)
    assert dec(ids) == "hello world"                                 # control symbols decode to nothing
    with pytest.raises(ValueError):
        SentencePieceEncoder(model, prefix_tokens=["<not a piece>"])
    # the native callable runs inside a pipeline's map step on worker threads
    texts = _corpus()[:64]
    plain = SentencePieceEncoder(model)
    out = list(read_sequence(texts).map(plain.native, num_parallel_calls=4).and_return())
    assert [t.tolist() for t in out] == [ref.EncodeAsIds(t) for t in texts]
    clone = pickle.loads(pickle.dumps(model))
    assert clone.encode("hello world") == model.encode("hello world") and clone.vocabulary_size == model.vocabulary_size


def test_malformed_models_are_refused(tmp_path, trained: dict[str, tuple]) -> None:
    blob = trained["unigram"][0].read_bytes()
    for name, data in (("empty", b""), ("cut", blob[: len(blob) // 2 + 1]), ("noise", bytes(range(256)) * 4)):
        bad = tmp_path / f"{name}.model"
        bad.write_bytes(data)
        with pytest.raises((ValueError, RuntimeError)):
            SentencePieceModel(bad)
    with pytest.raises((ValueError, RuntimeError)):
        SentencePieceModel(tmp_path / "absent.model")


def test_random_unicode_matches_the_package(trained: dict[str, tuple]) -> None:
    """Random code points from every UTF-8 length class, odd whitespace, literal control-symbol spellings."""
    rng = random.Random(1)

    def text() -> str:
        out = []
        for _ in range(rng.randint(0, 30)):
            r = rng.random()
            if r < 0.3:
                out.append(rng.choice("abcdefghijklmnopqrstuvwxyz ABC 012"))
            elif r < 0.4:
                out.append(rng.choice([" ", "  ", "\t", "\n", " ", "　", "​", "▁", "﻿", "­"]))
            elif r < 0.5:
                out.append(rng.choice(["<sep>", "<ctl>", "<s>", "</s>", "<unk>", "<0x41>"]))
            else:
                cp = 0xd800
                while 0xd800 <= cp <= 0xdfff:
                    cp = rng.choice([rng.randint(0, 0x7f), rng.randint(0x80, 0x7ff), rng.randint(0x800, 0xffff),
                                     rng.randint(0x10000, 0x10ffff)])
                out.append(chr(cp))
        return "".join(out)

    texts = [text() for _ in range(600)]
    for name in ("unigram", "bpe_byte_fallback", "unigram_case_folding", "bpe_keep_whitespace"):
        path, ref = trained[name]
        model = SentencePieceModel(path)
        for t in texts:
            ids = ref.EncodeAsIds(t)
            assert model.encode(t) == ids, (name, t)
            assert model.encode_as_tokens(t) == ref.EncodeAsPieces(t), (name, t)
            assert model.decode(ids) == ref.DecodeIds(ids), (name, t)
