"""Import stand-in for the reference's native package.

The reference's C++ runtime (data pipeline, audio/image decoders) cannot be
built offline because its third-party submodules are empty. The reference
itself supports running without it in "documentation mode", in which its data
modules define placeholders instead of importing the bindings. None of that is
on the model / FSDP / optimizer path that the benchmark's reference arm runs.
"""
DOC_MODE = True
__version__ = "0.9.0.dev0"


def get_lib():  # pragma: no cover - never used in DOC_MODE
    raise RuntimeError("fairseq2n is not available in this environment")


def get_include():  # pragma: no cover
    raise RuntimeError("fairseq2n is not available in this environment")


def get_cmake_prefix_path():  # pragma: no cover
    raise RuntimeError("fairseq2n is not available in this environment")


def supports_image() -> bool:
    return False


def supports_cuda() -> bool:
    return False


def cuda_version():
    return None
