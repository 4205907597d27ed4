"""Hot operators. Every op has two implementations:

* the hand-written sm_100a kernel from the in-tree extension ``fairseq2_b200._C``
  -- the only path taken for CUDA tensors (a missing extension on a GPU box is
  an error, never a silent fallback);
* a plain PyTorch fp32 formulation used for CPU tensors (plumbing tests over
  gloo) and as the numerical oracle of the kernel tests.
"""
from fairseq2_b200.ops._ext import ext_available, get_ext, require_ext  # noqa: F401
from fairseq2_b200.ops._ext import KernelWaitTimeout as KernelWaitTimeout
