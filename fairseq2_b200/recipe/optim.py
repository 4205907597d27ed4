"""Regex-selected optimizer parameter groups (cf. fairseq2 ``recipe/optim.py:33-232``).

``groups: [{params: "regex" | [regex...], lr: ..., weight_decay: ...}, ...]``:
each parameter joins the first group one of whose patterns fully matches its
name; the rest form the default group."""
from __future__ import annotations

import re
from typing import Any, Mapping, Sequence

from torch.nn import Module


def create_param_groups(module: Module, groups: Sequence[Mapping[str, Any]]) -> list[dict[str, Any]]:
    compiled = []
    for i, g in enumerate(groups):
        pats = g.get("params")
        if pats is None:
            raise ValueError(f"The optimizer group at index {i} must have a `params` field.")
        if isinstance(pats, str):
            pats = [pats]
        compiled.append(([re.compile(p) for p in pats], {k: v for k, v in g.items() if k != "params"}))
    buckets: list[list[Any]] = [[] for _ in compiled]
    rest = []
    for name, p in module.named_parameters():
        if not p.requires_grad:
            continue
        for i, (pats, _) in enumerate(compiled):
            if any(pt.fullmatch(name) for pt in pats):
                buckets[i].append(p)
                break
        else:
            rest.append(p)
    out = []
    for (pats, kw), ps in zip(compiled, buckets):
        if ps:
            d = dict(kw)
            if "betas" in d:
                d["betas"] = tuple(d["betas"])
            d["params"] = ps
            out.append(d)
    if rest:
        out.append({"params": rest})
    return out
