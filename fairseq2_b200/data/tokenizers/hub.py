"""Tokenizer families and ``load_tokenizer`` (cf. fairseq2
``data/tokenizers/family.py``, ``hub.py``)."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Callable

from fairseq2_b200.assets import AssetCard, AssetDownloadManager, AssetStore, get_asset_store
from fairseq2_b200.data.tokenizers.tokenizer import Tokenizer

TokenizerLoader = Callable[[Path, AssetCard], Tokenizer]

_families: dict[str, TokenizerLoader] = {}


class UnknownTokenizerFamilyError(LookupError):
    pass


def register_tokenizer_family(name: str, loader: TokenizerLoader) -> None:
    if name in _families:
        raise ValueError(f"The tokenizer family '{name}' is already registered.")
    _families[name] = loader


def _load_char(path: Path, card: AssetCard) -> Tokenizer:
    from fairseq2_b200.data.tokenizers.char import CharTokenizer

    return CharTokenizer()


def _load_sentencepiece(path: Path, card: AssetCard) -> Tokenizer:
    from fairseq2_b200.data.tokenizers.sentencepiece import BasicSentencePieceTokenizer

    return BasicSentencePieceTokenizer(path)


def _load_hg(path: Path, card: AssetCard) -> Tokenizer:
    from fairseq2_b200.data.tokenizers.hg import HuggingFaceTokenizer

    return HuggingFaceTokenizer(path)


def _load_llama(path: Path, card: AssetCard) -> Tokenizer:
    """tiktoken model file if present, otherwise the Hugging Face tokenizer in the same directory."""
    if path.is_file() and path.suffix in (".model", ".tiktoken"):
        from fairseq2_b200.data.tokenizers.tiktoken import TiktokenTokenizer

        return TiktokenTokenizer(path)
    cand = path / "original" / "tokenizer.model"
    if cand.exists() and not (path / "tokenizer.json").exists():
        from fairseq2_b200.data.tokenizers.tiktoken import TiktokenTokenizer

        return TiktokenTokenizer(cand)
    return _load_hg(path, card)


for _n, _l in (("char", _load_char), ("sentencepiece", _load_sentencepiece), ("hg", _load_hg), ("llama", _load_llama),
               ("qwen", _load_hg), ("mistral", _load_hg), ("olmo", _load_hg), ("gemma3n", _load_hg)):
    register_tokenizer_family(_n, _l)


def load_tokenizer(name_or_card: str | AssetCard, *, store: AssetStore | None = None,
                   download_manager: AssetDownloadManager | None = None) -> Tokenizer:
    store = store or get_asset_store()
    card = store.retrieve_card(name_or_card) if isinstance(name_or_card, str) else name_or_card
    family = card.maybe_get_field("tokenizer_family", str)
    if family is None:
        raise UnknownTokenizerFamilyError(f"The '{card.name}' asset card does not have a 'tokenizer_family' field.")
    loader = _families.get(family)
    if loader is None:
        raise UnknownTokenizerFamilyError(f"The tokenizer family '{family}' of '{card.name}' is not registered.")
    uri = card.maybe_get_field("tokenizer", str)
    if uri is None:
        path = Path(".")
    else:
        dm = download_manager or AssetDownloadManager()
        base = card.maybe_get_field("__base_path__", str)
        if base and "://" not in uri and not Path(uri).is_absolute():
            uri = str(Path(base) / uri)
        path = dm.download_tokenizer(uri, card.name)
    return loader(path, card)
