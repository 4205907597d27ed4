"""Chatbot abstractions (cf. fairseq2 ``recipes/chatbot/chatbot.py:23-101``, ``chatbot/llama.py:27-165``,
``chatbot/mistral.py``): a dialog is encoded with the model family's chat format and completed by a
sequence generator."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Literal, Sequence

import torch
from torch import Tensor

from fairseq2_b200.data.tokenizers import TokenDecoder, Tokenizer
from fairseq2_b200.generation import SequenceGenerator, SequenceGeneratorOutput
from fairseq2_b200.nn.batch_layout import BatchLayout


@dataclass
class Message:
    role: Literal["system", "user", "bot"]
    content: str


Dialog = Sequence[Message]


class DialogEncoder(ABC):
    @abstractmethod
    def encode(self, dialog: Dialog) -> Tensor: ...

    @property
    @abstractmethod
    def supports_system_prompt(self) -> bool: ...


def _check(dialog: Dialog) -> None:
    if len(dialog) == 0:
        raise ValueError("`dialog` must have at least one message with the 'user' role.")
    if dialog[-1].role != "user":
        raise ValueError("The last message of `dialog` must have the 'user' role.")


def _turns(dialog: Dialog):  # type: ignore[no-untyped-def]
    for user, bot in zip(dialog[::2], dialog[1::2]):
        if user.role != "user" or bot.role != "bot":
            raise ValueError("After an optional 'system' message, `dialog` must alternate between 'user' and 'bot'.")
        yield user, bot


class LLaMADialogEncoder(DialogEncoder):
    """LLaMA-2 chat format: ``<s>[INST] <<SYS>>...<</SYS>> user [/INST] bot</s>``."""

    def __init__(self, tokenizer: Tokenizer, device: torch.device) -> None:
        vi = tokenizer.vocab_info
        if vi.bos_idx is None or vi.eos_idx is None:
            raise ValueError("`tokenizer` must have BOS and EOS symbols defined.")
        self._bos = torch.tensor([vi.bos_idx], device=device)
        self._eos = torch.tensor([vi.eos_idx], device=device)
        self._enc = tokenizer.create_raw_encoder(device=device)

    def encode(self, dialog: Dialog) -> Tensor:
        _check(dialog)
        if dialog[0].role == "system":
            first = Message(dialog[1].role, f"<<SYS>>\n{dialog[0].content}\n<</SYS>>\n\n{dialog[1].content}")
            dialog = [first, *dialog[2:]]
        parts: list[Tensor] = []
        for user, bot in _turns(dialog):
            parts += [self._bos, self._enc(f"[INST] {user.content.strip()} [/INST] {bot.content.strip()}"), self._eos]
        parts += [self._bos, self._enc(f"[INST] {dialog[-1].content.strip()} [/INST]")]
        return torch.cat(parts)

    @property
    def supports_system_prompt(self) -> bool:
        return True


class LLaMA3DialogEncoder(DialogEncoder):
    """LLaMA-3 chat format with header tokens around the role names."""

    def __init__(self, tokenizer: Tokenizer, device: torch.device) -> None:
        vi = tokenizer.vocab_info
        if None in (vi.bos_idx, vi.eos_idx, vi.boh_idx, vi.eoh_idx):
            raise ValueError("`tokenizer` must have BOS, EOS, BOH and EOH symbols defined.")
        mk = lambda i: torch.tensor([i], device=device)  # noqa: E731
        self._bos, self._eos, self._boh, self._eoh = mk(vi.bos_idx), mk(vi.eos_idx), mk(vi.boh_idx), mk(vi.eoh_idx)
        self._enc = tokenizer.create_raw_encoder(device=device)
        self._break = self._enc("\n\n")

    def encode(self, dialog: Dialog) -> Tensor:
        _check(dialog)
        parts: list[Tensor] = [self._bos]

        def role(name: str) -> None:
            parts.extend([self._boh, self._enc(name), self._eoh, self._break])

        def content(text: str) -> None:
            parts.extend([self._enc(text.strip()), self._eos])

        if dialog[0].role == "system":
            role("system")
            content(dialog[0].content)
            dialog = dialog[1:]
        for user, bot in _turns(dialog):
            role("user")
            content(user.content)
            role("assistant")
            content(bot.content)
        role("user")
        content(dialog[-1].content)
        role("assistant")
        return torch.cat(parts)

    @property
    def supports_system_prompt(self) -> bool:
        return True


class MistralDialogEncoder(DialogEncoder):
    """``<s>[INST] user [/INST] bot</s>`` without a system prompt."""

    def __init__(self, tokenizer: Tokenizer, device: torch.device) -> None:
        vi = tokenizer.vocab_info
        if vi.bos_idx is None or vi.eos_idx is None:
            raise ValueError("`tokenizer` must have BOS and EOS symbols defined.")
        self._bos = torch.tensor([vi.bos_idx], device=device)
        self._eos = torch.tensor([vi.eos_idx], device=device)
        self._enc = tokenizer.create_raw_encoder(device=device)

    def encode(self, dialog: Dialog) -> Tensor:
        _check(dialog)
        parts: list[Tensor] = [self._bos]
        for user, bot in _turns(dialog):
            parts += [self._enc(f"[INST] {user.content.strip()} [/INST]"), self._enc(bot.content.strip()), self._eos]
        parts.append(self._enc(f"[INST] {dialog[-1].content.strip()} [/INST]"))
        return torch.cat(parts)

    @property
    def supports_system_prompt(self) -> bool:
        return False


def create_dialog_encoder(family: str, tokenizer: Tokenizer, device: torch.device) -> DialogEncoder:
    if family == "mistral":
        return MistralDialogEncoder(tokenizer, device)
    if family in ("llama", "llama4"):
        vi = tokenizer.vocab_info
        if vi.boh_idx is None and vi.eoh_idx is None:
            return LLaMADialogEncoder(tokenizer, device)
        return LLaMA3DialogEncoder(tokenizer, device)
    raise ValueError(f"The '{family}' model family has no chat format; supported: llama, llama4, mistral.")


class Chatbot(ABC):
    @abstractmethod
    def response(self, dialog: Dialog) -> tuple[Message, SequenceGeneratorOutput]: ...

    @property
    @abstractmethod
    def supports_system_prompt(self) -> bool: ...


class StandardChatbot(Chatbot):
    def __init__(self, generator: SequenceGenerator, dialog_encoder: DialogEncoder, text_decoder: TokenDecoder) -> None:
        self._generator, self._encoder, self._decoder = generator, dialog_encoder, text_decoder

    def response(self, dialog: Dialog) -> tuple[Message, SequenceGeneratorOutput]:
        seq = self._encoder.encode(dialog).unsqueeze(0)
        out = self._generator(seq, BatchLayout((1, seq.shape[1]), [seq.shape[1]], device=seq.device))
        hyps = out.hypotheses[0]
        if not hyps:
            raise RuntimeError("The sequence generator returned no hypothesis.")
        return Message("bot", self._decoder(hyps[0].seq)), out

    @property
    def supports_system_prompt(self) -> bool:
        return self._encoder.supports_system_prompt
