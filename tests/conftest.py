"""Test configuration: registers the ``gpu`` marker and skips GPU tests on
hosts without CUDA (they run with ``-m gpu`` on a B200)."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200 with `-m gpu`)")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def cuda() -> torch.device:
    return torch.device("cuda", 0)
