"""tiktoken-based tokenizer (LLaMA-3 style BPE files; cf. fairseq2
``data/tokenizers/tiktoken.py`` and ``models/llama/tokenizer.py``)."""
from __future__ import annotations

import base64
from pathlib import Path
from typing import Sequence

from torch import Tensor

from fairseq2_b200.data.tokenizers.tokenizer import (TokenDecoder, TokenEncoder, Tokenizer, VocabularyInfo,
                                                     _to_tensor)
from fairseq2_b200.typing import Device

_LLAMA3_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                 r"\s*[\r\n]+|\s+(?!\S)|\s+")


class TiktokenModel:
    def __init__(self, path: Path | str, split_regex: str = _LLAMA3_SPLIT, special_tokens: Sequence[str] | None = None,
                 num_prefix_special: int = 0) -> None:
        try:
            import tiktoken
        except ImportError as ex:
            raise RuntimeError("The `tiktoken` package is required for tiktoken tokenizers.") from ex
        ranks: dict[bytes, int] = {}
        with open(path, "rb") as fp:
            for line in fp:
                if not line.strip():
                    continue
                tok, rank = line.split()
                ranks[base64.b64decode(tok)] = int(rank)
        n = len(ranks)
        specials = {s: n + i for i, s in enumerate(special_tokens or [])}
        self.encoding = tiktoken.Encoding(name=Path(path).stem, pat_str=split_regex, mergeable_ranks=ranks,
                                          special_tokens=specials)
        self.special_tokens = specials
        self.size = n + len(specials)


class _TikEnc(TokenEncoder):
    def __init__(self, model: TiktokenModel, prefix: Sequence[int], suffix: Sequence[int], device: Device | None,
                 pin: bool) -> None:
        self._m, self._pre, self._suf, self._device, self._pin = model, list(prefix), list(suffix), device, pin

    def __call__(self, text: str) -> Tensor:
        ids = self._m.encoding.encode(text, allowed_special="all")
        return _to_tensor(self._pre + ids + self._suf, self._device, self._pin)

    def encode_as_tokens(self, text: str) -> list[str]:
        return [self._m.encoding.decode([i]) for i in self._m.encoding.encode(text, allowed_special="all")]


class _TikDec(TokenDecoder):
    def __init__(self, model: TiktokenModel, skip_special: bool) -> None:
        self._m, self._skip = model, skip_special
        self._special_ids = set(model.special_tokens.values())

    def __call__(self, token_indices: Tensor) -> str:
        ids = [int(i) for i in token_indices.tolist()]
        if self._skip:
            ids = [i for i in ids if i not in self._special_ids]
        return self._m.encoding.decode(ids)

    def decode_from_tokens(self, tokens: Sequence[str]) -> str:
        return "".join(tokens)


LLAMA3_SPECIAL_TOKENS = (["<|begin_of_text|>", "<|end_of_text|>", "<|reserved_special_token_0|>",
                          "<|reserved_special_token_1|>", "<|finetune_right_pad_id|>", "<|step_id|>",
                          "<|start_header_id|>", "<|end_header_id|>", "<|eom_id|>", "<|eot_id|>", "<|python_tag|>"]
                         + [f"<|reserved_special_token_{i}|>" for i in range(2, 247)])


class TiktokenTokenizer(Tokenizer):
    def __init__(self, path: Path | str, *, special_tokens: Sequence[str] = LLAMA3_SPECIAL_TOKENS,
                 bos_token: str = "<|begin_of_text|>", eos_token: str = "<|end_of_text|>",
                 pad_token: str | None = "<|finetune_right_pad_id|>") -> None:
        self._model = TiktokenModel(path, special_tokens=special_tokens)
        s = self._model.special_tokens
        self._bos, self._eos = s[bos_token], s[eos_token]
        self._pad = s.get(pad_token) if pad_token else None

    def create_encoder(self, *, task=None, lang=None, mode=None, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        table = {None: ([self._bos], [self._eos]), "default": ([self._bos], [self._eos]), "prompt": ([self._bos], []),
                 "prompt_response": ([], [self._eos]), "as_is": ([], [])}
        if mode not in table:
            raise ValueError(f"`mode` must be one of {[m for m in table if m]}, but is '{mode}' instead.")
        pre, suf = table[mode]
        return _TikEnc(self._model, pre, suf, device, pin_memory)

    def create_raw_encoder(self, *, device=None, pin_memory=False) -> TokenEncoder:  # type: ignore[no-untyped-def]
        return _TikEnc(self._model, [], [], device, pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> TokenDecoder:
        return _TikDec(self._model, skip_special_tokens)

    @property
    def vocab_info(self) -> VocabularyInfo:
        return VocabularyInfo(size=self._model.size, bos_idx=self._bos, eos_idx=self._eos, pad_idx=self._pad)
