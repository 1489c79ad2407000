"""B200-native CUDA backend for the decoder MoE layer of unlimitedocr.c.

The product is the C-ABI shared library built from csrc/ (see include/uocr_cuda_moe.h);
`ffi` binds it for Python callers.  The folder name is not a Python identifier, so import it
through `__graft_entry__.load_package()` or with importlib under any module name you like.
"""
from . import ep, ffi  # noqa: F401
from .ffi import Context, UocrCudaError, load_library  # noqa: F401
