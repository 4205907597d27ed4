"""Byte/character-level tokenizer: ids 0..3 are pad/bos/eos/unk, then one id per
UTF-8 byte. Needs no model file, so it is what the plumbing tests and the
synthetic recipes use."""
from __future__ import annotations

from typing import Sequence

from torch import Tensor

from fairseq2_b200.data.tokenizers.tokenizer import (TokenDecoder, TokenEncoder, Tokenizer, VocabularyInfo,
                                                     _to_tensor)
from fairseq2_b200.typing import Device

_OFFSET = 4


class _Enc(TokenEncoder):
    def __init__(self, bos: bool, eos: bool, device: Device | None, pin: bool) -> None:
        self._bos, self._eos, self._device, self._pin = bos, eos, device, pin

    def __call__(self, text: str) -> Tensor:
        ids = [b + _OFFSET for b in text.encode("utf-8")]
        if self._bos:
            ids.insert(0, 1)
        if self._eos:
            ids.append(2)
        return _to_tensor(ids, self._device, self._pin)

    def encode_as_tokens(self, text: str) -> list[str]:
        return [chr(b) if 32 <= b < 127 else f"<0x{b:02X}>" for b in text.encode("utf-8")]


class _Dec(TokenDecoder):
    def __call__(self, token_indices: Tensor) -> str:
        bs = bytes(int(i) - _OFFSET for i in token_indices.tolist() if _OFFSET <= int(i) < _OFFSET + 256)
        return bs.decode("utf-8", errors="replace")

    def decode_from_tokens(self, tokens: Sequence[str]) -> str:
        return "".join(tokens)


class CharTokenizer(Tokenizer):
    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        if mode in (None, "default"):
            return _Enc(True, True, device, pin_memory)
        if mode == "prompt":
            return _Enc(True, False, device, pin_memory)
        if mode == "prompt_response":
            return _Enc(False, True, device, pin_memory)
        if mode == "as_is":
            return _Enc(False, False, device, pin_memory)
        raise ValueError(f"`mode` must be 'default', 'prompt', 'prompt_response' or 'as_is', but is '{mode}' instead.")

    def create_raw_encoder(self, *, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        return _Enc(False, False, device, pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder:
        return _Dec()

    @property
    def vocab_info(self) -> VocabularyInfo:
        return VocabularyInfo(size=256 + _OFFSET, unk_idx=3, bos_idx=1, eos_idx=2, pad_idx=0)
