"""``pip install -e .`` builds the two native libraries in-tree (``fairseq2_b200/_C.so``: the sm_100a kernels,
``fairseq2_b200/_data.so``: the C++ data runtime) with the same code path as ``__graft_entry__.build()``.

The kernels need nvcc 12.8+ (``-gencode arch=compute_100a,code=sm_100a``); without nvcc only the data runtime is built
and the Python package still imports (CUDA ops then raise when they are first used)."""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self) -> None:
        root = Path(__file__).parent.resolve()
        sys.path.insert(0, str(root))
        try:
            from fairseq2_b200.csrc import build as native

            native.build_data()
            if shutil.which("nvcc") is not None:
                native.build_cuda()
            else:
                print("nvcc not found: skipping the sm_100a kernel extension", file=sys.stderr)
        finally:
            sys.path.pop(0)
        super().run()


setup(cmdclass={"build_py": BuildNative})
