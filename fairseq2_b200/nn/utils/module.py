"""Module helpers (cf. fairseq2 ``nn/utils/module.py:31-524``)."""
from __future__ import annotations

import re
from typing import Callable, Iterable, Iterator, Mapping, Sequence

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.gang import Gang
from fairseq2_b200.typing import Device


def reset_parameters(module: Module, *, recurse: bool = True) -> None:
    """Calls ``reset_parameters()`` on ``module`` and (optionally) its descendants, children first."""
    def visit(m: Module) -> None:
        if recurse:
            for c in m.children():
                visit(c)
        fn = getattr(m, "reset_parameters", None)
        if callable(fn):
            fn()

    visit(module)


def reset_non_persistent_buffers(module: Module, *, recurse: bool = True) -> None:
    def visit(m: Module) -> None:
        if recurse:
            for c in m.children():
                visit(c)
        fn = getattr(m, "reset_non_persistent_buffers", None)
        if callable(fn):
            fn()

    visit(module)


def to_device(module: Module, device: Device) -> None:
    module.to(device)


def to_empty(module: Module, device: Device, *, recurse: bool = True) -> None:
    """Materialises meta parameters/buffers on ``device`` without initialising them.
    Parameters that are shared between modules stay shared."""
    memo: dict[int, Tensor] = {}

    def conv(t: Tensor) -> Tensor:
        key = id(t)
        if key not in memo:
            memo[key] = torch.empty_like(t, device=device)
        return memo[key]

    def visit(m: Module) -> None:
        for name, p in list(m._parameters.items()):
            if p is None:
                continue
            key = id(p)
            if key in memo:
                m._parameters[name] = memo[key]  # type: ignore[assignment]
                continue
            np_ = Parameter(torch.empty_like(p, device=device), requires_grad=p.requires_grad)
            memo[key] = np_
            m._parameters[name] = np_
        for name, b in list(m._buffers.items()):
            if b is not None:
                m._buffers[name] = conv(b)
        if recurse:
            for c in m.children():
                visit(c)

    visit(module)


def apply_to_parameters(module: Module, fn: Callable[[Tensor], Tensor], *, recurse: bool = True,
                        no_memo: bool = False) -> None:
    memo: dict[int, Tensor] = {}

    def run(t: Tensor) -> Tensor:
        if no_memo:
            return fn(t)
        k = id(t)
        if k not in memo:
            memo[k] = fn(t)
        return memo[k]

    def visit(m: Module) -> None:
        for name, p in list(m._parameters.items()):
            if p is None:
                continue
            with torch.no_grad():
                new = run(p)
            if new is not p:
                m._parameters[name] = Parameter(new, requires_grad=p.requires_grad) if not isinstance(new, Parameter) else new
        for name, b in list(m._buffers.items()):
            if b is not None:
                m._buffers[name] = run(b)
        if recurse:
            for c in m.children():
                visit(c)

    visit(module)


def freeze_parameters(module: Module | None, value: bool = True) -> None:
    if module is None:
        return
    module.requires_grad_(not value)


def select_parameters(module: Module, names: Sequence[str], *, exclude: bool = False
                      ) -> Iterator[tuple[str, Parameter]]:
    """Parameters whose fully-qualified name fully matches any regex in ``names``."""
    pats = [re.compile(n) for n in names]
    for name, p in module.named_parameters():
        hit = any(pt.fullmatch(name) for pt in pats)
        if hit != exclude:
            yield name, p


def share_parameters(source: Module, target: Module) -> None:
    """Makes ``target`` use the very same Parameter objects as ``source``."""
    src = dict(source.named_parameters())
    tgt = dict(target.named_parameters())
    if src.keys() != tgt.keys():
        raise ValueError("`source` and `target` must have the same parameter names.")
    for name, p in src.items():
        mod = target
        *path, leaf = name.split(".")
        for part in path:
            mod = getattr(mod, part)
        mod._parameters[leaf] = p


def broadcast_module(module: Module, gang: Gang, *, source_rank: int = 0, bucket_bytes: int = 250 * 1024 * 1024,
                     skip_buffers: bool = False) -> None:
    """Broadcasts parameters (and buffers) from ``source_rank`` in coalesced
    buckets of ``bucket_bytes``."""
    if gang.size == 1:
        return
    tensors: list[Tensor] = []
    seen: set[int] = set()
    items: Iterable[Tensor] = list(module.parameters()) + ([] if skip_buffers else list(module.buffers()))
    for t in items:
        if id(t) in seen or t.device.type == "meta":
            continue
        seen.add(id(t))
        tensors.append(t.detach())
    by_dtype: dict[torch.dtype, list[Tensor]] = {}
    for t in tensors:
        by_dtype.setdefault(t.dtype, []).append(t)
    for dt, ts in by_dtype.items():
        bucket: list[Tensor] = []
        size = 0

        def flush() -> None:
            nonlocal bucket, size
            if not bucket:
                return
            flat = torch.cat([b.reshape(-1) for b in bucket])
            gang.broadcast(flat, source_rank)
            off = 0
            for b in bucket:
                n = b.numel()
                b.copy_(flat[off: off + n].view_as(b))
                off += n
            bucket, size = [], 0

        for t in ts:
            nbytes = t.numel() * t.element_size()
            if size + nbytes > bucket_bytes and bucket:
                flush()
            bucket.append(t)
            size += nbytes
        flush()


def load_state_dict(module: Module, state_dict: Mapping[str, object], *, strict: bool = True) -> None:
    """``Module.load_state_dict`` that also reports keys belonging to modules
    that are set to ``None`` on this instance."""
    res = module.load_state_dict(state_dict, strict=False)  # type: ignore[arg-type]
    if strict and (res.missing_keys or res.unexpected_keys):
        msg = []
        if res.missing_keys:
            msg.append(f"missing keys: {sorted(res.missing_keys)}")
        if res.unexpected_keys:
            msg.append(f"unexpected keys: {sorted(res.unexpected_keys)}")
        raise ValueError("`state_dict` does not match the module: " + "; ".join(msg))


def get_module_size(module: Module) -> tuple[int, int, int]:
    """(param_count, trainable_param_count, param_bytes)."""
    n = tr = nb = 0
    for p in module.parameters():
        n += p.numel()
        nb += p.numel() * p.element_size()
        if p.requires_grad:
            tr += p.numel()
    return n, tr, nb


def infer_device(module: Module) -> Device:
    devs = {p.device for p in module.parameters()} | {b.device for b in module.buffers()}
    if len(devs) > 1:
        raise ValueError(f"All parameters and buffers of `module` must be on one device, but are on {sorted(map(str, devs))}.")
    return devs.pop() if devs else torch.device("cpu")
