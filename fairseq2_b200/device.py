"""Current/default device handling (cf. ``src/fairseq2/device.py``).

The default device is ``FAIRSEQ2_DEVICE`` if set, else ``cuda:LOCAL_RANK`` when
CUDA is present, else CPU. ``set_device`` is a thread-local context stack that
also installs the device as torch's default device for factory functions.
"""
from __future__ import annotations

import os
import threading
from contextlib import contextmanager
from typing import Iterator, Mapping

import torch

from fairseq2_b200.typing import Device

CPU = torch.device("cpu")
META_DEVICE = torch.device("meta")

_tls = threading.local()
_default_device: Device | None = None


class DeviceDetectionError(Exception):
    pass


def detect_default_device(env: Mapping[str, str] | None = None) -> Device:
    env = os.environ if env is None else env
    s = env.get("FAIRSEQ2_DEVICE")
    if s is not None:
        try:
            return torch.device(s)
        except (RuntimeError, ValueError):
            raise DeviceDetectionError(
                f"`FAIRSEQ2_DEVICE` environment variable must be a device string, but is '{s}' instead.") from None
    if torch.cuda.is_available() and torch.cuda.device_count() > 0:
        n = torch.cuda.device_count()
        try:
            idx = int(env.get("LOCAL_RANK", "0"))
        except ValueError:
            raise DeviceDetectionError("`LOCAL_RANK` environment variable must be an integer.") from None
        if idx >= n:
            raise DeviceDetectionError(
                f"`LOCAL_RANK` ({idx}) must be less than the number of CUDA devices ({n}).")
        return torch.device("cuda", idx)
    return CPU


def get_default_device() -> Device:
    global _default_device
    if _default_device is None:
        _default_device = detect_default_device()
        if _default_device.type == "cuda":
            torch.cuda.set_device(_default_device)
    return _default_device


def set_default_device(device: Device | None) -> None:
    global _default_device
    _default_device = device


def get_current_device() -> Device:
    stack = getattr(_tls, "stack", None)
    if stack:
        return stack[-1]
    return get_default_device()


@contextmanager
def set_device(device: Device) -> Iterator[None]:
    stack = getattr(_tls, "stack", None)
    if stack is None:
        stack = _tls.stack = []
    stack.append(device)
    try:
        with device:
            yield
    finally:
        stack.pop()
