"""SentencePiece-based tokenizers (basic, NLLB, S2T) and the tokenizer / model hubs, on a tiny model trained here."""
from __future__ import annotations

from pathlib import Path

import pytest
import torch

spm = pytest.importorskip("sentencepiece")

from fairseq2_b200.data.tokenizers.hub import get_tokenizer_hub  # noqa: E402
from fairseq2_b200.data.tokenizers.sentencepiece import (BasicSentencePieceTokenizer, NllbTokenizer,  # noqa: E402
                                                         S2TTransformerTokenizer, SentencePieceModel)

_TEXT = ["the quick brown fox jumps over the lazy dog", "pack my box with five dozen liquor jugs",
         "how vexingly quick daft zebras jump", "sphinx of black quartz judge my vow"] * 8


@pytest.fixture(scope="module")
def spm_path(tmp_path_factory: pytest.TempPathFactory) -> Path:
    d = tmp_path_factory.mktemp("spm")
    corpus = d / "corpus.txt"
    corpus.write_text("\n".join(_TEXT))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(d / "tiny"), vocab_size=64, model_type="bpe",
                                   user_defined_symbols=["<lang:de>", "<lang:fr>"], minloglevel=2)
    return d / "tiny.model"


def test_basic_modes_and_round_trip(spm_path: Path) -> None:
    tok = BasicSentencePieceTokenizer(spm_path)
    vi = tok.vocab_info
    assert vi.size == 64 and vi.unk_idx == 0 and vi.bos_idx == 1 and vi.eos_idx == 2 and vi.pad_idx is None
    ids = tok.create_encoder()("the quick fox")
    assert ids.dtype == torch.int64 and int(ids[0]) == vi.bos_idx and int(ids[-1]) == vi.eos_idx
    raw = tok.create_raw_encoder()("the quick fox")
    assert ids[1:-1].tolist() == raw.tolist()
    assert int(tok.create_encoder(mode="prompt")("the")[-1]) != vi.eos_idx
    assert tok.create_decoder()(ids) == "the quick fox"
    with pytest.raises(ValueError):
        tok.create_encoder(mode="nope")


def test_front_inserted_symbol_shifts_every_piece(spm_path: Path) -> None:
    plain = SentencePieceModel(spm_path)
    shifted = SentencePieceModel(spm_path, control_symbols=["__eng__", "<pad>@0"])
    assert shifted.pad_idx == 0 and shifted.token_to_index("<pad>") == 0 and shifted.index_to_token(0) == "<pad>"
    assert shifted.encode("lazy dog") == [i + 1 for i in plain.encode("lazy dog")]
    assert shifted.token_to_index("</s>") == plain.token_to_index("</s>") + 1
    vi = shifted.vocab_info
    assert vi.pad_idx == 0 and vi.unk_idx == 1 and vi.bos_idx == 2 and vi.eos_idx == 3 and vi.size == 64 + 1 + 1
    assert shifted.token_to_index("__eng__") == 65 and shifted.index_to_token(65) == "__eng__"
    assert shifted.decode(shifted.encode("lazy dog") + [0, 65]) == "lazy dog"


def test_nllb_source_and_target_framing(spm_path: Path) -> None:
    tok = NllbTokenizer(spm_path, ["eng_Latn", "deu_Latn"], "eng_Latn")
    m = tok._model
    eos, eng, deu = m.token_to_index("</s>"), m.token_to_index("__eng_Latn__"), m.token_to_index("__deu_Latn__")
    src = tok.create_encoder()("lazy dog").tolist()
    assert src[0] == eng and src[-1] == eos and eos not in src[:-1]
    tgt = tok.create_encoder(lang="deu_Latn", mode="target")("lazy dog").tolist()
    assert tgt[:2] == [eos, deu] and tgt[-1] == eos
    mined = tok.create_encoder(mode="source_mining")("lazy dog").tolist()
    assert mined[:2] == [eng, m.token_to_index("<MINED_DATA>")]
    assert tok.vocab_info.pad_idx == 0 and tok.vocab_info.size == 64 + 1 + 2 + 3
    assert tok.create_decoder()(torch.tensor(tgt)) == "lazy dog"
    with pytest.raises(ValueError):
        tok.create_encoder(lang="fra_Latn")
    with pytest.raises(ValueError):
        tok.create_encoder(task="transcription")


def test_s2t_target_prefix(spm_path: Path) -> None:
    multi = S2TTransformerTokenizer(spm_path, "translation", ["de", "fr"], "de")
    m = multi._model
    ids = multi.create_encoder(lang="fr")("lazy dog").tolist()
    assert ids[:2] == [m.token_to_index("</s>"), m.token_to_index("<lang:fr>")]
    mono = S2TTransformerTokenizer(spm_path, "transcription", ["en"], "en")
    assert mono.create_encoder()("lazy dog").tolist()[0] == m.token_to_index("</s>")
    assert len(mono.create_encoder()("lazy dog")) == len(ids) - 1
    with pytest.raises(ValueError):
        mono.create_encoder(task="translation")
    with pytest.raises(ValueError):
        S2TTransformerTokenizer(spm_path, "summarization")


def test_tokenizer_hub_custom_load(spm_path: Path) -> None:
    hub = get_tokenizer_hub("nllb")
    tok = hub.load_custom_tokenizer(spm_path, {"langs": ["eng_Latn", "fra_Latn"], "default_lang": "fra_Latn"})
    assert isinstance(tok, NllbTokenizer) and tok.default_lang == "fra_Latn"
    assert isinstance(get_tokenizer_hub("sentencepiece").load_custom_tokenizer(spm_path), BasicSentencePieceTokenizer)
    with pytest.raises(LookupError):
        get_tokenizer_hub("no_such_family")


def test_model_hub_accessors() -> None:
    from fairseq2_b200.models import hub

    assert "llama3_8b" in hub.get_llama_model_hub().get_archs()
    for name in ("llama4", "mistral", "qwen", "olmo", "gemma3n", "nllb", "s2t_transformer", "s2t_conformer",
                 "wav2vec2", "wav2vec2_asr", "w2vbert", "jepa", "jepa_classifier", "hg"):
        h = getattr(hub, f"get_{name}_model_hub")()
        assert isinstance(h.get_archs(), list), name


def test_tokenizer_ref_is_followed() -> None:
    from fairseq2_b200.assets import AssetStore
    from fairseq2_b200.assets.store import InMemoryAssetMetadataProvider
    from fairseq2_b200.data.tokenizers.char import CharTokenizer
    from fairseq2_b200.data.tokenizers.hub import load_tokenizer, resolve_tokenizer_reference

    provider = InMemoryAssetMetadataProvider([
        {"name": "tok_card", "tokenizer_family": "char"},
        {"name": "model_a", "model_family": "wav2vec2_asr", "tokenizer_ref": "tok_card"},
        {"name": "model_b", "tokenizer_ref": "model_a"},
        {"name": "loop_a", "tokenizer_ref": "loop_b"},
        {"name": "loop_b", "tokenizer_ref": "loop_a"},
        {"name": "dangling", "tokenizer_ref": "nowhere"},
    ])
    store = AssetStore([provider])
    assert resolve_tokenizer_reference(store, store.retrieve_card("model_b")).name == "tok_card"
    assert isinstance(load_tokenizer("model_b", store=store), CharTokenizer)
    with pytest.raises(LookupError, match="cycle"):
        load_tokenizer("loop_a", store=store)
    with pytest.raises(LookupError, match="does not exist"):
        load_tokenizer("dangling", store=store)
