"""SentencePiece tokenizers over the ``sentencepiece`` runtime (cf. fairseq2
``data/tokenizers/sentencepiece.py:19-110``): ``SentencePieceModel`` with extra
control symbols, encoder with prefix/suffix tokens, sampling and reversal,
decoder."""
from __future__ import annotations

from pathlib import Path
from typing import Sequence

from torch import Tensor

from fairseq2_b200.data.tokenizers.tokenizer import (TokenDecoder, TokenEncoder, Tokenizer, VocabularyInfo,
                                                     _to_tensor)
from fairseq2_b200.typing import Device


class SentencePieceModel:
    """A SentencePiece model with extra control symbols.

    A symbol that the model does not know is appended after the model's pieces. A symbol written ``"<sym>@0"`` is
    instead INSERTED at index 0 and every piece of the model moves up by one (the reference's native model does the
    same for NLLB, whose SentencePiece model has no pad symbol: fairseq2 ``models/nllb/tokenizer.py:149-159``)."""

    def __init__(self, path: Path | str, control_symbols: Sequence[str] | None = None) -> None:
        try:
            import sentencepiece as spm
        except ImportError as ex:
            raise RuntimeError("The `sentencepiece` package is required for SentencePiece tokenizers.") from ex
        self._sp = spm.SentencePieceProcessor()
        self._sp.Load(str(path))
        base = self._sp.GetPieceSize()
        self._front: str | None = None
        for s in control_symbols or []:
            if s.endswith("@0"):
                if self._front is not None:
                    raise ValueError("Only one control symbol can be inserted at index 0.")
                self._front = s[:-2]
        self._shift = 0 if self._front is None else 1
        self._extra: dict[str, int] = {}
        for s in control_symbols or []:
            if s.endswith("@0"):
                continue
            idx = self._sp.PieceToId(s)
            known = idx != self._sp.unk_id() or s == self._sp.IdToPiece(self._sp.unk_id())
            if not known and s not in self._extra:
                self._extra[s] = self._shift + base + len(self._extra)
        self._extra_by_index = {i: s for s, i in self._extra.items()}

    @property
    def processor(self):  # type: ignore[no-untyped-def]
        return self._sp

    @property
    def index_shift(self) -> int:
        """What is added to the model's own piece indices (1 if a symbol was inserted at index 0)."""
        return self._shift

    def encode(self, text: str, **kwargs: object) -> list[int]:
        ids = self._sp.Encode(text, **kwargs)
        return [int(i) + self._shift for i in ids] if self._shift else [int(i) for i in ids]

    def decode(self, indices: Sequence[int]) -> str:
        n, sh = self._sp.GetPieceSize(), self._shift
        return str(self._sp.Decode([i - sh for i in indices if sh <= i < n + sh]))

    def token_to_index(self, token: str) -> int:
        if token == self._front:
            return 0
        if token in self._extra:
            return self._extra[token]
        return int(self._sp.PieceToId(token)) + self._shift

    def index_to_token(self, idx: int) -> str:
        if idx == 0 and self._front is not None:
            return self._front
        if idx in self._extra_by_index:
            return self._extra_by_index[idx]
        return str(self._sp.IdToPiece(idx - self._shift))

    @property
    def vocab_info(self) -> VocabularyInfo:
        sp, sh = self._sp, self._shift

        def opt(i: int) -> int | None:
            return i + sh if i >= 0 else None

        pad = 0 if self._front is not None else opt(sp.pad_id())
        return VocabularyInfo(size=sp.GetPieceSize() + sh + len(self._extra), unk_idx=opt(sp.unk_id()),
                              bos_idx=opt(sp.bos_id()), eos_idx=opt(sp.eos_id()), pad_idx=pad)


def load_sentencepiece_model(path: Path | str, control_symbols: Sequence[str] | None = None) -> SentencePieceModel:
    return SentencePieceModel(path, control_symbols)


class SentencePieceEncoder(TokenEncoder):
    def __init__(self, model: SentencePieceModel, *, prefix_tokens: Sequence[str] | None = None,
                 suffix_tokens: Sequence[str] | None = None, reverse: bool = False, enable_sampling: bool = False,
                 nbest_size: int = -1, alpha: float = 0.1, device: Device | None = None, pin_memory: bool = False) -> None:
        self._m = model
        self._prefix = [model.token_to_index(t) for t in (prefix_tokens or [])]
        self._suffix = [model.token_to_index(t) for t in (suffix_tokens or [])]
        self._reverse, self._sampling, self._nbest, self._alpha = reverse, enable_sampling, nbest_size, alpha
        self._device, self._pin = device, pin_memory

    def __call__(self, text: str) -> Tensor:
        ids = self._m.encode(text, enable_sampling=self._sampling, nbest_size=self._nbest, alpha=self._alpha)
        if self._reverse:
            ids = ids[::-1]
        return _to_tensor(self._prefix + list(ids) + self._suffix, self._device, self._pin)

    def encode_as_tokens(self, text: str) -> list[str]:
        toks = self._m.processor.EncodeAsPieces(text)
        return toks[::-1] if self._reverse else toks


class SentencePieceDecoder(TokenDecoder):
    def __init__(self, model: SentencePieceModel, reverse: bool = False) -> None:
        self._m, self._reverse = model, reverse

    def __call__(self, token_indices: Tensor) -> str:
        ids = [int(i) for i in token_indices.tolist()]
        if self._reverse:
            ids = ids[::-1]
        return self._m.decode(ids)

    def decode_from_tokens(self, tokens: Sequence[str]) -> str:
        return str(self._m.processor.DecodePieces(list(tokens)))


class BasicSentencePieceTokenizer(Tokenizer):
    """BOS ... EOS in default mode; prompt: BOS only; prompt_response: EOS only; as_is: neither."""

    def __init__(self, path: Path | str) -> None:
        self._model = SentencePieceModel(path)

    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        table = {None: (["<s>"], ["</s>"]), "default": (["<s>"], ["</s>"]), "prompt": (["<s>"], []),
                 "prompt_response": ([], ["</s>"]), "as_is": ([], [])}
        if mode not in table:
            raise ValueError(f"`mode` must be one of {[m for m in table if m]}, but is '{mode}' instead.")
        pre, suf = table[mode]
        return SentencePieceEncoder(self._model, prefix_tokens=pre, suffix_tokens=suf, device=device,
                                    pin_memory=pin_memory)

    def create_raw_encoder(self, *, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        return SentencePieceEncoder(self._model, device=device, pin_memory=pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder:
        return SentencePieceDecoder(self._model)

    @property
    def vocab_info(self) -> VocabularyInfo:
        return self._model.vocab_info


RawSentencePieceTokenizer = BasicSentencePieceTokenizer


class NllbTokenizer(Tokenizer):
    """NLLB: a language token replaces BOS in source sequences, target sequences start with EOS and the language
    token (cf. fairseq2 ``models/nllb/tokenizer.py:33-135``)."""

    _SOURCE_MODES = {"source": [], "source_mining": ["<MINED_DATA>"], "source_mmt_bt": ["<MMT_BT_DATA>"],
                     "source_smt_bt": ["<SMT_BT_DATA>"]}

    def __init__(self, path: Path | str, langs: Sequence[str], default_lang: str) -> None:
        symbols = [f"__{lang}__" for lang in langs] + ["<MINED_DATA>", "<MMT_BT_DATA>", "<SMT_BT_DATA>", "<pad>@0"]
        self._model = SentencePieceModel(path, control_symbols=symbols)
        self._langs, self._default_lang = set(langs), default_lang

    @property
    def langs(self) -> set[str]:
        return self._langs

    @property
    def default_lang(self) -> str:
        return self._default_lang

    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        if task is not None and task != "translation":
            raise ValueError(f"`task` must be 'translation', but is '{task}' instead.")
        lang = lang or self._default_lang
        if lang not in self._langs:
            raise ValueError(f"`lang` must be a supported language, but is '{lang}' instead.")
        mode = mode or "source"
        if mode in self._SOURCE_MODES:
            prefix = [f"__{lang}__", *self._SOURCE_MODES[mode]]
        elif mode == "target":
            prefix = ["</s>", f"__{lang}__"]
        else:
            raise ValueError(f"`mode` must be 'source' or 'target', but is '{mode}' instead.")
        return SentencePieceEncoder(self._model, prefix_tokens=prefix, suffix_tokens=["</s>"], device=device,
                                    pin_memory=pin_memory)

    def create_raw_encoder(self, *, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        return SentencePieceEncoder(self._model, device=device, pin_memory=pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder:
        return SentencePieceDecoder(self._model)

    @property
    def vocab_info(self) -> VocabularyInfo:
        return self._model.vocab_info


class S2TTransformerTokenizer(Tokenizer):
    """Speech-to-text targets: EOS first, then ``<lang:xx>`` for multilingual translation (cf. fairseq2
    ``models/s2t_transformer/tokenizer.py:32-131``)."""

    def __init__(self, path: Path | str, task: str = "translation", target_langs: Sequence[str] = ("en",),
                 default_target_lang: str = "en") -> None:
        if task not in ("transcription", "translation"):
            raise ValueError(f"`task` must be 'transcription' or 'translation', but is '{task}' instead.")
        self._model = SentencePieceModel(path)
        self._task, self._target_langs, self._default = task, set(target_langs), default_target_lang

    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        if task is not None and task != self._task:
            raise ValueError(f"`task` must be '{self._task}', but is '{task}' instead.")
        if mode is not None and mode != "target":
            raise ValueError(f"`mode` must be 'target', but is '{mode}' instead.")
        lang = lang or self._default
        if lang not in self._target_langs:
            raise ValueError(f"`lang` must be a supported language, but is '{lang}' instead.")
        prefix = ["</s>"]
        if self._task == "translation" and len(self._target_langs) > 1:
            prefix.append(f"<lang:{lang}>")
        return SentencePieceEncoder(self._model, prefix_tokens=prefix, device=device, pin_memory=pin_memory)

    def create_raw_encoder(self, *, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        return SentencePieceEncoder(self._model, device=device, pin_memory=pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder:
        return SentencePieceDecoder(self._model)

    @property
    def vocab_info(self) -> VocabularyInfo:
        return self._model.vocab_info
