"""Hugging Face tokenizers (cf. fairseq2 ``data/tokenizers/hg.py:126-208``),
including ``apply_chat_template`` used by chat-mode SFT."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Sequence

from torch import Tensor

from fairseq2_b200.data.tokenizers.tokenizer import (TokenDecoder, TokenEncoder, Tokenizer, VocabularyInfo,
                                                     _to_tensor)
from fairseq2_b200.typing import Device


class HuggingFaceTokenEncoder(TokenEncoder):
    def __init__(self, tok: Any, *, add_bos: bool, add_eos: bool, device: Device | None, pin_memory: bool) -> None:
        self._tok, self._bos, self._eos, self._device, self._pin = tok, add_bos, add_eos, device, pin_memory

    def __call__(self, text: str) -> Tensor:
        ids = self._tok.encode(text, add_special_tokens=False)
        if self._bos and self._tok.bos_token_id is not None:
            ids = [self._tok.bos_token_id] + ids
        if self._eos and self._tok.eos_token_id is not None:
            ids = ids + [self._tok.eos_token_id]
        return _to_tensor(ids, self._device, self._pin)

    def encode_as_tokens(self, text: str) -> list[str]:
        return list(self._tok.tokenize(text))

    def apply_chat_template(self, messages: Sequence[dict[str, str]], *, add_generation_prompt: bool = False) -> Tensor:
        ids = self._tok.apply_chat_template(list(messages), tokenize=True, add_generation_prompt=add_generation_prompt)
        return _to_tensor(ids, self._device, self._pin)


class HuggingFaceTokenDecoder(TokenDecoder):
    def __init__(self, tok: Any, skip_special_tokens: bool) -> None:
        self._tok, self._skip = tok, skip_special_tokens

    def __call__(self, token_indices: Tensor) -> str:
        return str(self._tok.decode(token_indices.tolist(), skip_special_tokens=self._skip))

    def decode_from_tokens(self, tokens: Sequence[str]) -> str:
        return str(self._tok.convert_tokens_to_string(list(tokens)))


class HuggingFaceTokenizer(Tokenizer):
    def __init__(self, path: Path | str, **kwargs: Any) -> None:
        try:
            from transformers import AutoTokenizer
        except ImportError as ex:
            raise RuntimeError("The `transformers` package is required for Hugging Face tokenizers.") from ex
        self._tok = AutoTokenizer.from_pretrained(str(path), **kwargs)

    @property
    def raw(self) -> Any:
        return self._tok

    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        table = {None: (True, True), "default": (True, True), "prompt": (True, False),
                 "prompt_response": (False, True), "as_is": (False, False)}
        if mode not in table:
            raise ValueError(f"`mode` must be one of {[m for m in table if m]}, but is '{mode}' instead.")
        b, e = table[mode]
        return HuggingFaceTokenEncoder(self._tok, add_bos=b, add_eos=e, device=device, pin_memory=pin_memory)

    def create_raw_encoder(self, *, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        return HuggingFaceTokenEncoder(self._tok, add_bos=False, add_eos=False, device=device, pin_memory=pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder:
        return HuggingFaceTokenDecoder(self._tok, skip_special_tokens)

    @property
    def vocab_info(self) -> VocabularyInfo:
        t = self._tok
        return VocabularyInfo(size=len(t), unk_idx=t.unk_token_id, bos_idx=t.bos_token_id, eos_idx=t.eos_token_id,
                              pad_idx=t.pad_token_id)
