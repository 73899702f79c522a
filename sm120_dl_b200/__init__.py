"""B200 (sm_100a) kernels for the two hot paths of HugeOrca/sm120-dl.

The product is the C ABI library libb200dl.so (include/b200dl.h) plus host code that mirrors
the reference's own interfaces: the GEMM config registry and `test_gemm_cute` harness
(gemm/), and the `flashatten_v3_sm120` Python module (flashattention/).  This package
exposes the same entry points to Python through ctypes.  There is no CPU or PyTorch
fallback: importing `ops` without the built library raises ImportError.
"""

from . import capi  # noqa: F401

__all__ = ["capi"]
