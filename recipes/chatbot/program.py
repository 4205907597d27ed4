"""Interactive chat program (cf. fairseq2 ``recipes/chatbot/program.py:30-190``, ``chatbot/cli.py``).

Rank 0 talks to the user and broadcasts every message to the other (tensor-parallel) ranks so that all of
them run the same generation; the reply is streamed piece by piece through a generator step hook.

    python -m recipes.chatbot --model llama3_2_1b_instruct
    torchrun --nproc-per-node 2 -m recipes.chatbot --model llama3_1_70b_instruct --tensor-parallel-size 2
"""
from __future__ import annotations

import argparse
import sys
from abc import ABC, abstractmethod
from datetime import timedelta
from typing import Any

import torch
from torch import Tensor

from fairseq2_b200.assets import get_asset_store
from fairseq2_b200.data.tokenizers import TokenDecoder, load_tokenizer
from fairseq2_b200.device import get_default_device
from fairseq2_b200.gang import Gang, create_parallel_gangs, setup_root_gang
from fairseq2_b200.generation import SamplingSequenceGenerator, SequenceGenerator, TopPSampler
from fairseq2_b200.models.family import get_model_family

from .chatbot import Chatbot, Message, StandardChatbot, create_dialog_encoder


class ProgramView(ABC):
    @abstractmethod
    def input_system_prompt(self) -> str: ...

    @abstractmethod
    def input_message(self) -> str: ...

    @abstractmethod
    def print_reply(self, message: str) -> None: ...

    @abstractmethod
    def print_reply_piece(self, piece: str) -> None: ...


class ConsoleView(ProgramView):
    def __init__(self, model_name: str) -> None:
        self._name = model_name

    def input_system_prompt(self) -> str:
        return input("System Prompt (press enter to skip): ")

    def input_message(self) -> str:
        return input("\nYou> ")

    def print_reply(self, message: str) -> None:
        print(f"\n{self._name}> {message}", end="", flush=True)

    def print_reply_piece(self, piece: str) -> None:
        print(piece, end="", flush=True)


class MessagePrintHook:
    """Prints only the text that the latest decoding step added."""

    def __init__(self, view: ProgramView, text_decoder: TokenDecoder, prompt_len: int) -> None:
        self._view, self._decode, self._prompt_len = view, text_decoder, prompt_len
        self._first, self._prev_len = True, 0

    def __call__(self, prompt_indices: Tensor, seqs: Tensor, step_scores: Tensor | None, prefill: bool) -> None:
        if prefill or len(prompt_indices) != 1:
            return
        text = self._decode(seqs[0, self._prompt_len:])
        if len(text) == self._prev_len:
            return
        piece = text[self._prev_len:]
        self._prev_len = len(text)
        if self._first:
            piece = piece.lstrip()
            if not piece:
                return
            self._first = False
        self._view.print_reply_piece(piece)


class ChatbotProgram:
    def __init__(self, view: ProgramView, chatbot: Chatbot, generator: SequenceGenerator, tokenizer: Any,
                 gang: Gang, dialog_encoder: Any) -> None:
        self._view, self._chatbot, self._generator, self._tokenizer = view, chatbot, generator, tokenizer
        self._gang, self._encoder = gang, dialog_encoder
        self._dialog: list[Message] = []

    def run(self) -> None:
        if self._gang.rank == 0:
            self._run_interactive()
        else:
            self._run_non_interactive()

    def _share(self, message: Message) -> None:
        self._dialog.append(message)
        self._gang.broadcast_objects([message])

    def _run_interactive(self) -> None:
        if self._chatbot.supports_system_prompt:
            prompt = self._view.input_system_prompt()
            if prompt:
                self._share(Message("system", prompt))
        while True:
            text = self._view.input_message()
            if text == "bye":
                break
            self._share(Message("user", text))
            self._view.print_reply("")
            decoder = self._tokenizer.create_decoder(skip_special_tokens=True)
            prompt_len = int(self._encoder.encode(self._dialog).numel())
            with self._generator.register_step_hook(MessagePrintHook(self._view, decoder, prompt_len)):
                response, _ = self._chatbot.response(self._dialog)
            self._view.print_reply_piece("\n")
            self._dialog.append(response)
        self._gang.broadcast_objects([Message("user", "bye")])
        self._view.print_reply("Bye!\n")

    def _run_non_interactive(self) -> None:
        while True:
            buf: list[Any] = [None]
            self._gang.broadcast_objects(buf)
            msg = buf[0]
            if not isinstance(msg, Message):
                raise RuntimeError(f"The received object is of type `{type(msg)}`.")
            if msg.content == "bye" and msg.role == "user":
                break
            self._dialog.append(msg)
            if msg.role == "system":
                continue
            response, _ = self._chatbot.response(self._dialog)
            self._dialog.append(response)


def main(argv: list[str] | None = None, view: ProgramView | None = None) -> int:
    ap = argparse.ArgumentParser(description="Chat with an instruction-tuned model.")
    ap.add_argument("--model", default="llama3_2_1b_instruct", help="model (asset card) name")
    ap.add_argument("--tokenizer", default=None, help="tokenizer name (defaults to the model name)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--top-p", type=float, default=0.8)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--max-gen-len", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=2)
    args = ap.parse_args(argv)
    torch.manual_seed(args.seed)
    device = get_default_device()
    root = setup_root_gang(device, timeout=timedelta(minutes=999))
    gangs = create_parallel_gangs(root, tp_size=args.tensor_parallel_size)
    if gangs.dp.size > 1:
        print("The world size must equal --tensor-parallel-size.", file=sys.stderr)
        return 2
    store = get_asset_store()
    card = store.retrieve_card(args.model)
    family = get_model_family(card.get_field("model_family", str))
    model = family.load_model(card, gangs, getattr(torch, args.dtype), store=store).eval()
    tokenizer = load_tokenizer(args.tokenizer or args.model, store=store)
    vi = tokenizer.vocab_info
    generator = SamplingSequenceGenerator(model, vi.eos_idx, vi.pad_idx, TopPSampler(args.top_p),
                                          temperature=args.temperature, max_gen_len=args.max_gen_len)
    encoder = create_dialog_encoder(family.name, tokenizer, device)
    chatbot = StandardChatbot(generator, encoder, tokenizer.create_decoder(skip_special_tokens=True))
    ChatbotProgram(view or ConsoleView(args.model), chatbot, generator, tokenizer, gangs.root, encoder).run()
    root.close()
    return 0
