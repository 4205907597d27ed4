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


def _load_nllb(path: Path, card: AssetCard) -> Tokenizer:
    from fairseq2_b200.data.tokenizers.sentencepiece import NllbTokenizer

    cfg = card.maybe_get_field("tokenizer_config") or {}
    langs = list(cfg.get("langs") or card.maybe_get_field("langs") or ["eng_Latn"])
    default = cfg.get("default_lang") or card.maybe_get_field("default_lang") or langs[0]
    return NllbTokenizer(path, langs, default)


def _load_s2t_transformer(path: Path, card: AssetCard) -> Tokenizer:
    from fairseq2_b200.data.tokenizers.sentencepiece import S2TTransformerTokenizer

    cfg = card.maybe_get_field("tokenizer_config") or {}
    return S2TTransformerTokenizer(path, cfg.get("task", "translation"), list(cfg.get("target_langs", ["en"])),
                                   cfg.get("default_target_lang", "en"))


for _n, _l in (("nllb", _load_nllb), ("s2t_transformer", _load_s2t_transformer), ("llama4", _load_llama),
               ("char", _load_char), ("sentencepiece", _load_sentencepiece), ("hg", _load_hg), ("llama", _load_llama),
               ("qwen", _load_hg), ("mistral", _load_hg), ("olmo", _load_hg), ("gemma3n", _load_hg)):
    register_tokenizer_family(_n, _l)


def resolve_tokenizer_reference(store: AssetStore, card: AssetCard) -> AssetCard:
    """Follows ``tokenizer_ref`` fields (a model card that names the card of its tokenizer) to the card that holds the
    tokenizer itself (cf. fairseq2 ``data/tokenizers/ref.py:12-33``)."""
    first, seen = card.name, {card.name}
    while True:
        ref = card.maybe_get_field("tokenizer_ref", str)
        if ref is None:
            return card
        if ref in seen:
            raise UnknownTokenizerFamilyError(f"The `tokenizer_ref` fields starting at '{first}' form a cycle at '{ref}'.")
        seen.add(ref)
        try:
            card = store.retrieve_card(ref)
        except LookupError:
            raise UnknownTokenizerFamilyError(
                f"The '{ref}' asset referenced by the '{first}' asset card does not exist.") from None


def load_tokenizer(name_or_card: str | AssetCard, *, store: AssetStore | None = None,
                   download_manager: AssetDownloadManager | None = None) -> Tokenizer:
    store = store or get_asset_store()
    card = store.retrieve_card(name_or_card) if isinstance(name_or_card, str) else name_or_card
    card = resolve_tokenizer_reference(store, card)
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


class TokenizerHub:
    """Typed accessor of one tokenizer family (cf. fairseq2 ``data/tokenizers/hub.py``): cards of the family,
    ``load_tokenizer`` by card name, ``load_custom_tokenizer`` from a path."""

    def __init__(self, family: str, store: AssetStore | None = None) -> None:
        if family not in _families:
            raise UnknownTokenizerFamilyError(f"The tokenizer family '{family}' is not registered.")
        self._family, self._store = family, store

    @property
    def family(self) -> str:
        return self._family

    def iter_cards(self):  # type: ignore[no-untyped-def]
        store = self._store or get_asset_store()
        for name in store.retrieve_names():
            card = store.retrieve_card(name)
            if card.maybe_get_field("tokenizer_family", str) == self._family:
                yield card

    def load_tokenizer(self, name_or_card: str | AssetCard) -> Tokenizer:
        store = self._store or get_asset_store()
        card = store.retrieve_card(name_or_card) if isinstance(name_or_card, str) else name_or_card
        family = card.maybe_get_field("tokenizer_family", str)
        if family != self._family:
            raise UnknownTokenizerFamilyError(
                f"The '{card.name}' tokenizer belongs to the '{family}' family, not to '{self._family}'.")
        return load_tokenizer(card, store=store)

    def load_custom_tokenizer(self, path: Path, config: dict[str, Any] | None = None) -> Tokenizer:
        card = AssetCard("custom", {"name": "custom", "tokenizer_family": self._family,
                                    "tokenizer_config": dict(config or {})})
        return _families[self._family](Path(path), card)


def get_tokenizer_hub(family: str) -> TokenizerHub:
    return TokenizerHub(family)
