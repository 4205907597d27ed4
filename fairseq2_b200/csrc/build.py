"""Builds the in-tree native extensions.

``python -m fairseq2_b200.csrc.build`` compiles

* ``fairseq2_b200/_C.so``    -- the sm_100a CUDA kernels (``-gencode
  arch=compute_100a,code=sm_100a``; nvcc cross-compiles without a GPU), and
* ``fairseq2_b200/_data.so`` -- the C++ data pipeline runtime (host only),

with ``torch.utils.cpp_extension`` + ninja and leaves the shared objects next
to the Python package so they are importable without installation.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent

CUDA_SOURCES = ["bindings.cpp", "gemm_tcgen05.cu", "elementwise.cu", "attention.cu", "comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
              "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__"]


def _newer(srcs: list[Path], target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    deps = list(srcs) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((CSRC / "data").glob("*.h"))
    return any(s.stat().st_mtime > t for s in deps)


def build_cuda(verbose: bool = False, force: bool = False) -> Path:
    from torch.utils import cpp_extension

    target = PKG / "_C.so"
    sources = [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]
    extra = sorted(p for p in CSRC.glob("*.cu") if p.name not in CUDA_SOURCES)
    sources += extra
    if not force and not _newer(sources, target):
        return target
    build_dir = CSRC / "_build" / "cuda"
    build_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(min(os.cpu_count() or 4, 16)))
    cpp_extension.load(name="_C", sources=[str(s) for s in sources], extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=NVCC_FLAGS,
                       # the C++ runtime is named explicitly: the toolchain's link driver leaves it out of DT_NEEDED,
                       # and the extension would then bind `__cxa_throw` and friends to whichever copy the process
                       # happens to have loaded first
                       extra_ldflags=["-l:libstdc++.so.6"],
                       build_directory=str(build_dir), verbose=verbose, is_python_module=False,
                       with_cuda=True)
    shutil.copy2(build_dir / "_C.so", target)
    return target


def build_data(verbose: bool = False, force: bool = False) -> Path | None:
    from torch.utils import cpp_extension

    src_dir = CSRC / "data"
    sources = sorted(src_dir.glob("*.cc")) if src_dir.exists() else []
    if not sources:
        return None
    target = PKG / "_data.so"
    if not force and not _newer(sources, target):
        return target
    # FAIRSEQ2_B200_SANITIZE=address|undefined|thread builds the data runtime with that sanitizer into
    # _data_<kind>.so (load it with LD_PRELOAD of the sanitizer runtime); the regular build is untouched
    sanitize = os.environ.get("FAIRSEQ2_B200_SANITIZE", "")
    if sanitize and sanitize not in ("address", "undefined", "thread"):
        raise ValueError(f"FAIRSEQ2_B200_SANITIZE must be address, undefined or thread, but is '{sanitize}'.")
    cflags, ldflags, tag = ["-O2", "-std=c++17", "-pthread"], ["-pthread", "-lz", "-l:libstdc++.so.6"], "data"
    if sanitize:
        cflags += [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-g"]
        ldflags += [f"-fsanitize={sanitize}"]
        tag = f"data_{sanitize}"
        target = PKG / f"_data_{sanitize}.so"
    build_dir = CSRC / "_build" / tag
    build_dir.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(name="_data", sources=[str(s) for s in sources], extra_cflags=cflags, extra_ldflags=ldflags,
                       build_directory=str(build_dir), verbose=verbose, is_python_module=False, with_cuda=False)
    shutil.copy2(build_dir / "_data.so", target)
    return target


def build_data_tests(verbose: bool = False, force: bool = False) -> Path | None:
    """``_data_tests.so``: the data runtime's sources (without the Python bindings) plus the C++ unit tests of
    ``csrc/data/tests``; ``run_all()`` of that module returns one row per test case."""
    from torch.utils import cpp_extension

    src_dir = CSRC / "data"
    tests = sorted((src_dir / "tests").glob("*.cc")) if (src_dir / "tests").exists() else []
    if not tests:
        return None
    sources = [s for s in sorted(src_dir.glob("*.cc")) if s.name != "bindings.cc"] + tests
    target = PKG / "_data_tests.so"
    if not force and not _newer(sources, target):
        return target
    build_dir = CSRC / "_build" / "data_tests"
    build_dir.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(name="_data_tests", sources=[str(s) for s in sources],
                       extra_cflags=["-O1", "-std=c++17", "-pthread"], extra_ldflags=["-pthread", "-lz", "-l:libstdc++.so.6"],
                       build_directory=str(build_dir), verbose=verbose, is_python_module=False, with_cuda=False)
    shutil.copy2(build_dir / "_data_tests.so", target)
    return target


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_cuda(verbose=verbose, force=force)
    build_data(verbose=verbose, force=force)
    build_data_tests(verbose=verbose, force=force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print("built:", [str(p) for p in PKG.glob("*.so")])
