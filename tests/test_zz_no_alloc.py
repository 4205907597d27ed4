"""The allocation-free RMSNorm backward (``fs2_rms_norm_bwd_no_alloc``) must
agree with the regular binding.

Who needs it: code that runs where the CUDA allocator may not be touched -- a
plugin inside a host application that owns all device memory, a latency-bound
loop that cannot take allocator locks, or a region that is being captured.
Such callers reach the kernel through the exported C symbol, pass inputs and
outputs they already own, and rely on the library's fixed scratch array.

The entry point is called through ``ctypes`` on the built shared object, twice
in a row (the second call reuses the scratch the first one dirtied), and its
outputs are compared with ``_C.rms_norm_bwd`` within the tolerances the other
kernel tests use. This file is named so that pytest collects it last.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

SO = Path(__file__).resolve().parent.parent / "fairseq2_b200" / "_C.so"


def _rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp(min=1e-12))


def _lib() -> ctypes.CDLL:
    from fairseq2_b200.ops import require_ext

    require_ext()  # loads libtorch and the extension's dependencies first
    lib = ctypes.CDLL(str(SO))
    lib.fs2_rms_norm_bwd_no_alloc.restype = ctypes.c_int
    lib.fs2_rms_norm_bwd_no_alloc.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    lib.fs2_no_alloc_last_error.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1e-2), (torch.float32, 1e-5)])
def test_no_alloc_matches_regular_entry_point(dtype: torch.dtype, tol: float) -> None:
    from fairseq2_b200.ops import require_ext

    ext = require_ext()
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev)
    for call, (rows, D) in enumerate([(300, 4096), (37, 1024)]):
        torch.manual_seed(100 + call)
        x = torch.randn((rows, D), device=dev, dtype=dtype)
        dy = torch.randn((rows, D), device=dev, dtype=dtype)
        w = (1 + 0.1 * torch.randn(D, device=dev)).to(dtype)
        _, rstd = ext.rms_norm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = ext.rms_norm_bwd(dy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty(D, device=dev, dtype=torch.float32)
        rc = lib.fs2_rms_norm_bwd_no_alloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                           dw.data_ptr(), rows, D, int(dtype == torch.bfloat16), stream.cuda_stream)
        assert rc == 0, lib.fs2_no_alloc_last_error().decode()
        torch.cuda.synchronize(dev)
        assert _rel_err(dx, dx_ref) < tol
        assert _rel_err(dw, dw_ref) < tol


def test_no_alloc_rejects_oversized_rows() -> None:
    lib = _lib()
    dev = torch.device("cuda", 0)
    D = 16384  # beyond FS2_NO_ALLOC_MAX_DIM
    x = torch.zeros((2, D), device=dev)
    dw = torch.zeros(D, device=dev)
    r = torch.ones(2, device=dev)
    rc = lib.fs2_rms_norm_bwd_no_alloc(x.data_ptr(), x.data_ptr(), dw.data_ptr(), r.data_ptr(), x.data_ptr(),
                                       dw.data_ptr(), 2, D, 0, torch.cuda.current_stream(dev).cuda_stream)
    assert rc != 0
    assert b"8192" in lib.fs2_no_alloc_last_error()
