"""argparse helpers: ``--config key=value`` action and a ``torch.dtype`` argument type.

``ConfigAction`` turns ``a.b=1 set:c.d={x: 2} del:e.f`` into the overlay mapping the config merger understands:
plain and ``set:`` items become ``{"a": {"_set_": {"b": 1}}}`` (replace the key wholesale), ``del:`` items become
``{"e": {"_del_": ["f"]}}``. Each use of the option appends one overlay to ``namespace.<dest>``
(fairseq2 ``utils/argparse.py:27-142``).
"""

from __future__ import annotations

from argparse import ZERO_OR_MORE, Action, ArgumentError, ArgumentParser, ArgumentTypeError, Namespace
from typing import Any

import torch

from fairseq2_b200.utils.yaml import YamlError, parse_yaml_value


def _parent_node(root: dict[str, Any], path: str) -> tuple[dict[str, Any], str]:
    *parents, leaf = path.split(".")
    node = root
    for key in parents:
        child = node.get(key)
        if not isinstance(child, dict):
            child = node[key] = {}
        node = child
    return node, leaf


class ConfigAction(Action):
    def __init__(self, option_strings: list[str], dest: str, help: str | None = None) -> None:
        super().__init__(option_strings, nargs=ZERO_OR_MORE, help=help, metavar="NAME=VALUE", dest=dest)

    def __call__(self, parser: ArgumentParser, namespace: Namespace, values: Any, option_string: str | None = None) -> None:
        overlay: dict[str, Any] = {}
        for raw in values:
            item = raw.strip()
            if item.startswith("del:"):
                path = item[4:]
                if "=" in path:
                    raise ArgumentError(self, f"key should not contain '=': {item}")
                node, leaf = _parent_node(overlay, path)
                node.setdefault("_del_", []).append(leaf)
                continue
            path, sep, text = item.partition("=")
            if not sep:
                raise ArgumentError(self, f"invalid key-value pair: {item}")
            try:
                value = parse_yaml_value(text.lstrip())
            except YamlError:
                raise ArgumentError(self, f"invalid key-value pair: {item} (value must be yaml)") from None
            path = path.rstrip()
            if path.startswith("set:"):
                path = path[4:]
            node, leaf = _parent_node(overlay, path)
            node.setdefault("_set_", {})[leaf] = value
        overlays = getattr(namespace, self.dest, None) or []
        overlays.append(overlay)
        setattr(namespace, self.dest, overlays)


def parse_dtype(value: str) -> torch.dtype:
    """``"bfloat16"`` or ``"torch.bfloat16"`` -> ``torch.bfloat16``."""
    dtype = getattr(torch, value.removeprefix("torch."), None)
    if not isinstance(dtype, torch.dtype):
        raise ArgumentTypeError("must be a torch.dtype identifier")
    return dtype
