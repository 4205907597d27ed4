"""Version helpers (cf. ``src/fairseq2/utils/version.py``)."""
from __future__ import annotations

import torch
from packaging.version import Version


def torch_greater_or_equal(major: int, minor: int) -> bool:
    v = Version(torch.__version__.split("+")[0])
    return (v.major, v.minor) >= (major, minor)
