"""SentencePiece tokenizers on the native runtime of the data pipeline (``csrc/data/sentencepiece.cc``: model reader,
normalizer, unigram / BPE / character / word segmentation; no dependency on the ``sentencepiece`` package).
Cf. fairseq2 ``data/tokenizers/sentencepiece.py:19-110``: ``SentencePieceModel`` with extra control symbols, encoder
with prefix/suffix tokens, sampling and reversal, decoder. Encoders and decoders are native callables, so a
``DataPipeline.map`` runs them on its worker threads without the interpreter lock."""
from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch
from torch import Tensor

from fairseq2_b200.data.tokenizers.tokenizer import TokenDecoder, TokenEncoder, Tokenizer, VocabularyInfo
from fairseq2_b200.typing import Device


def _native():  # type: ignore[no-untyped-def]
    from fairseq2_b200.data.data_pipeline import _n

    return _n


class SentencePieceModel:
    """A SentencePiece model with extra control symbols.

    A symbol that the model does not know is appended after the model's pieces as a control piece. A symbol written
    ``"<sym>@0"`` is instead INSERTED at index 0, every piece of the model moves up by one, and the symbol becomes
    the pad symbol (the reference's native model does the same for NLLB, whose SentencePiece model has no pad
    symbol: fairseq2 ``models/nllb/tokenizer.py:149-159``)."""

    def __init__(self, path: Path | str, control_symbols: Sequence[str] | None = None) -> None:
        self._path = str(path)
        self._control_symbols = list(control_symbols or [])
        self._m = _native().SentencePieceModel(self._path, self._control_symbols)

    def __getstate__(self) -> dict[str, object]:
        return {"path": self._path, "control_symbols": self._control_symbols}

    def __setstate__(self, state: dict[str, object]) -> None:
        self.__init__(state["path"], state["control_symbols"])  # type: ignore[misc, arg-type]

    @property
    def native(self):  # type: ignore[no-untyped-def]
        return self._m

    def encode(self, text: str) -> list[int]:
        return list(self._m.encode(text))

    def encode_as_tokens(self, text: str) -> list[str]:
        return list(self._m.encode_as_tokens(text))

    def nbest_encode(self, text: str, nbest_size: int) -> list[tuple[list[int], float]]:
        """The ``nbest_size`` best segmentations of a unigram model with their scores, best first."""
        return [(list(ids), float(score)) for ids, score in self._m.nbest_encode(text, nbest_size)]

    def decode(self, indices: Sequence[int]) -> str:
        n = self._m.vocabulary_size
        return str(self._m.decode([int(i) for i in indices if 0 <= int(i) < n]))

    def decode_from_tokens(self, tokens: Sequence[str]) -> str:
        return str(self._m.decode_from_tokens(list(tokens)))

    def normalize(self, text: str) -> str:
        return str(self._m.normalize(text))

    def token_to_index(self, token: str) -> int:
        return int(self._m.token_to_index(token))

    def index_to_token(self, idx: int) -> str:
        return str(self._m.index_to_token(idx))

    @property
    def vocabulary_size(self) -> int:
        return int(self._m.vocabulary_size)

    @property
    def unk_idx(self) -> int | None:
        return self._m.unk_idx

    @property
    def bos_idx(self) -> int | None:
        return self._m.bos_idx

    @property
    def eos_idx(self) -> int | None:
        return self._m.eos_idx

    @property
    def pad_idx(self) -> int | None:
        return self._m.pad_idx

    @property
    def vocab_info(self) -> VocabularyInfo:
        m = self._m
        return VocabularyInfo(size=m.vocabulary_size, unk_idx=m.unk_idx, bos_idx=m.bos_idx, eos_idx=m.eos_idx,
                              pad_idx=m.pad_idx)


def load_sentencepiece_model(path: Path | str, control_symbols: Sequence[str] | None = None) -> SentencePieceModel:
    return SentencePieceModel(path, control_symbols)


class SentencePieceEncoder(TokenEncoder):
    """``enable_sampling``: unigram models sample a segmentation (``nbest_size`` < 0: from all of them, with inverse
    temperature ``alpha``; > 1: among the n best), BPE models drop merges with probability ``alpha``. The sampler is
    seeded from the CPU generator, so ``torch.manual_seed`` makes it repeatable."""

    def __init__(self, model: SentencePieceModel, *, prefix_tokens: Sequence[str] | None = None,
                 suffix_tokens: Sequence[str] | None = None, reverse: bool = False, enable_sampling: bool = False,
                 nbest_size: int = -1, alpha: float = 0.1, device: Device | None = None, pin_memory: bool = False) -> None:
        seed = int(torch.randint(0, 2**62, (1,), device="cpu")) if enable_sampling else 0
        self._e = _native().SentencePieceEncoder(
            model.native, list(prefix_tokens or []), list(suffix_tokens or []), reverse, enable_sampling, nbest_size,
            alpha, None if device is None else str(device), pin_memory, seed)

    @property
    def native(self):  # type: ignore[no-untyped-def]
        """The native callable: hand it to ``DataPipelineBuilder.map`` to tokenize on the worker threads."""
        return self._e

    def __call__(self, text: str) -> Tensor:
        return self._e(text)

    def encode_as_tokens(self, text: str) -> list[str]:
        return list(self._e.encode_as_tokens(text))


class SentencePieceDecoder(TokenDecoder):
    def __init__(self, model: SentencePieceModel, reverse: bool = False) -> None:
        self._m, self._reverse = model, reverse

    def __call__(self, token_indices: Tensor) -> str:
        if token_indices.dim() != 1:
            raise ValueError(
                f"The input tensor must be one dimensional, but has {token_indices.dim()} dimension(s) instead.")
        if token_indices.dtype not in (torch.int16, torch.int32, torch.int64):
            raise ValueError("`sp_decoder` supports only `torch.int16`, `torch.int32`, and `torch.int64` data types.")
        ids = [int(i) for i in token_indices.tolist()]
        if self._reverse:
            ids = ids[::-1]
        return self._m.decode(ids)

    def decode_from_tokens(self, tokens: Sequence[str]) -> str:
        tokens = list(tokens)
        return self._m.decode_from_tokens(tokens[::-1] if self._reverse else tokens)


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
