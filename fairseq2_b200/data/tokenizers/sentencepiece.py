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
    def __init__(self, path: Path | str, control_symbols: Sequence[str] | None = None) -> None:
        try:
            import sentencepiece as spm
        except ImportError as ex:
            raise RuntimeError("The `sentencepiece` package is required for SentencePiece tokenizers.") from ex
        self._sp = spm.SentencePieceProcessor()
        self._sp.Load(str(path))
        self._extra: dict[str, int] = {}
        base = self._sp.GetPieceSize()
        for i, s in enumerate(control_symbols or []):
            if s.endswith("@0"):      # "<pad>@0" style: symbol takes over index 0 (fairseq convention)
                self._extra[s[:-2]] = 0
            else:
                idx = self._sp.PieceToId(s)
                self._extra[s] = idx if idx != self._sp.unk_id() else base + len(self._extra)

    @property
    def processor(self):  # type: ignore[no-untyped-def]
        return self._sp

    def token_to_index(self, token: str) -> int:
        if token in self._extra:
            return self._extra[token]
        return int(self._sp.PieceToId(token))

    def index_to_token(self, idx: int) -> str:
        for s, i in self._extra.items():
            if i == idx:
                return s
        return str(self._sp.IdToPiece(idx))

    @property
    def vocab_info(self) -> VocabularyInfo:
        sp = self._sp
        size = sp.GetPieceSize() + sum(1 for i in self._extra.values() if i >= sp.GetPieceSize())

        def opt(i: int) -> int | None:
            return i if i >= 0 else None

        return VocabularyInfo(size=size, unk_idx=opt(sp.unk_id()), bos_idx=opt(sp.bos_id()), eos_idx=opt(sp.eos_id()),
                              pad_idx=opt(sp.pad_id()))


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
        ids = self._m.processor.Encode(text, enable_sampling=self._sampling, nbest_size=self._nbest, alpha=self._alpha)
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
        n = self._m.processor.GetPieceSize()
        return str(self._m.processor.Decode([i for i in ids if 0 <= i < n]))

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
