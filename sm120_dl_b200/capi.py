"""ctypes binding of the C ABI in include/b200dl.h (libb200dl.so).

This is the only way Python code in this package reaches the kernels.  There is no
fallback: if the library is missing or a call fails, an exception is raised.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200dl.so")

B200_OK = 0


class B200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"b200dl error {code}: {message}")
        self.code = code


class GemmConfig(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("bm", ctypes.c_int), ("bn", ctypes.c_int),
                ("bk", ctypes.c_int), ("stages", ctypes.c_int), ("cta_group", ctypes.c_int),
                ("acc_bufs", ctypes.c_int), ("bs_w", ctypes.c_int), ("smem_bytes", ctypes.c_int),
                ("tmem_cols", ctypes.c_int), ("split_k", ctypes.c_int)]


class FaConfig(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("head_dim", ctypes.c_int), ("block_m", ctypes.c_int),
                ("block_n", ctypes.c_int), ("tile_q", ctypes.c_int), ("q_tiles", ctypes.c_int),
                ("tile_kv", ctypes.c_int), ("stages", ctypes.c_int), ("nwarps", ctypes.c_int),
                ("smem_bytes", ctypes.c_int), ("softmax_layout", ctypes.c_int)]


EXPORTS = (
    "b200_gemm_num_configs", "b200_gemm_get_config", "b200_gemm_find_config",
    "b200_gemm_default_config", "b200_gemm_set_stream_k", "b200_gemm_uses_stream_k",
    "b200_gemm_bf16_tn", "b200_gemm_f16_tn", "b200_gemm_bf16_tn_noalloc", "b200_gemm_noalloc_status",
    "b200_gemm_bf16_tn_scatter",
    "b200_fa_num_configs", "b200_fa_get_config", "b200_fa_find_config",
    "b200_fa_default_config", "b200_fa_fwd_fp16", "b200_fa_fwd_fp16_scatter",
    "b200_last_error", "b200_device_status", "b200_selftest_wait_expiry", "b200_version",
)

_lib = None


def lib():
    """Load libb200dl.so (once) and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sm120_dl_b200.build lib` "
            "(there is no CPU or PyTorch fallback)")
    L = ctypes.CDLL(LIB_PATH)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    i64p = ctypes.POINTER(ctypes.c_int64)
    L.b200_gemm_num_configs.restype = ctypes.c_int
    L.b200_gemm_get_config.restype = ctypes.POINTER(GemmConfig)
    L.b200_gemm_get_config.argtypes = [ctypes.c_int]
    L.b200_gemm_find_config.restype = ctypes.c_int
    L.b200_gemm_find_config.argtypes = [ctypes.c_char_p]
    L.b200_gemm_default_config.restype = ctypes.c_int
    L.b200_gemm_default_config.argtypes = [ctypes.c_int] * 3
    L.b200_gemm_set_stream_k.restype = ctypes.c_int
    L.b200_gemm_set_stream_k.argtypes = [ctypes.c_int]
    L.b200_gemm_uses_stream_k.restype = ctypes.c_int
    L.b200_gemm_uses_stream_k.argtypes = [ctypes.c_int] * 4
    L.b200_gemm_bf16_tn.restype = ctypes.c_int
    L.b200_gemm_bf16_tn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                    vp, i64, vp, i64, vp, i64, vp]
    L.b200_gemm_f16_tn.restype = ctypes.c_int
    L.b200_gemm_f16_tn.argtypes = L.b200_gemm_bf16_tn.argtypes
    L.b200_gemm_bf16_tn_scatter.restype = ctypes.c_int
    L.b200_gemm_bf16_tn_scatter.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, i64, vp, i64,
                                            ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, i64, vp]
    L.b200_gemm_bf16_tn_noalloc.restype = ctypes.c_int
    L.b200_gemm_bf16_tn_noalloc.argtypes = L.b200_gemm_bf16_tn.argtypes
    L.b200_gemm_noalloc_status.restype = ctypes.c_int
    L.b200_gemm_noalloc_status.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    if not hasattr(L, "b200_fa_fwd_fp16"):
        raise ImportError(f"{LIB_PATH} does not export the attention entry points; rebuild it")
    L.b200_fa_num_configs.restype = ctypes.c_int
    L.b200_fa_get_config.restype = ctypes.POINTER(FaConfig)
    L.b200_fa_get_config.argtypes = [ctypes.c_int]
    L.b200_fa_find_config.restype = ctypes.c_int
    L.b200_fa_find_config.argtypes = [ctypes.c_char_p]
    L.b200_fa_default_config.restype = ctypes.c_int
    L.b200_fa_default_config.argtypes = [ctypes.c_int]
    L.b200_fa_fwd_fp16.restype = ctypes.c_int
    L.b200_fa_fwd_fp16.argtypes = [ctypes.c_int, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int,
                                   ctypes.c_int, ctypes.c_int, ctypes.c_int, i64p, i64p, i64p,
                                   i64p, ctypes.c_float, ctypes.c_int, vp]
    L.b200_fa_fwd_fp16_scatter.restype = ctypes.c_int
    L.b200_fa_fwd_fp16_scatter.argtypes = [ctypes.c_int, vp, vp, vp, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           i64p, i64p, i64p, i64p, ctypes.c_float, ctypes.c_int, vp]
    L.b200_last_error.restype = ctypes.c_char_p
    L.b200_device_status.restype = ctypes.c_int
    L.b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    L.b200_selftest_wait_expiry.restype = ctypes.c_int
    L.b200_selftest_wait_expiry.argtypes = [ctypes.c_uint32, vp]
    L.b200_version.restype = ctypes.c_char_p
    _lib = L
    return L


def check(rc):
    if rc != B200_OK:
        raise B200Error(rc, lib().b200_last_error().decode())


def _cfg_dict(struct):
    d = {}
    for name, _ in struct._fields_:
        val = getattr(struct, name)
        d[name] = val.decode() if isinstance(val, bytes) else val
    return d


def gemm_configs():
    L = lib()
    return [_cfg_dict(L.b200_gemm_get_config(i).contents) for i in range(L.b200_gemm_num_configs())]


def fa_configs():
    L = lib()
    return [_cfg_dict(L.b200_fa_get_config(i).contents) for i in range(L.b200_fa_num_configs())]


def noalloc_status():
    """Synchronise the current device; return the status word of the allocation-free GEMM's
    built-in scratch array (0 = its last launch ran to completion)."""
    code = ctypes.c_uint32(0)
    check(lib().b200_gemm_noalloc_status(ctypes.byref(code)))
    return code.value


def device_status():
    """Synchronise the current device; return its kernel status word (0 = healthy)."""
    code = ctypes.c_uint32(0)
    check(lib().b200_device_status(ctypes.byref(code)))
    return code.value
