"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the cpu_baseline / reference legs of bench.py may import
this module; the product package never does.

Two layers:
  * `gemm_f64`, `attention_f32`, `compare`: ctypes calls into liboracle.so (oracle.cpp,
    OpenMP), usable at the benchmark's full sizes or on row subsets of them;
  * `gemm_numpy`, `attention_numpy`: independent numpy float64 restatements used to pin
    the C++ code on small cases.

Parity status: "parity unpinned" with respect to reference-held vectors -- the reference
(HugeOrca/sm120-dl) stores none; its checks are run-time comparisons against cuBLAS
(gemm/test.cpp:394-420) and flash-attn (flashattention/v3_mMnNkN/verify.py:129).  The
oracle is pinned to numpy float64 / torch CPU results through tests/golden/.

Semantics restated (reference file:line):
  GEMM       C = A @ B.T with A [M,K], B [N,K] (gemm/gemm_cute.hpp:302-304)
  attention  softmax(Q K^T / sqrt(D)) V on [B,S,H,D] (kernel_traits.hpp:146-160,
             pybind/flash_fwd_config.cu.in:27), causal mask row < col
             (flashatten_v3.hpp:101-103)
  compare    |got-ref| <= abs + rel*|ref| (gemm/test.cpp:165-230; verify.py:64-80)
"""

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "oracle.cpp"))):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        i64p = ctypes.POINTER(ctypes.c_int64)
        L.oracle_num_threads.restype = ctypes.c_int
        L.oracle_set_num_threads.restype = None
        L.oracle_set_num_threads.argtypes = [ctypes.c_int]
        L.oracle_gemm_bf16_tn_f64.restype = None
        L.oracle_gemm_bf16_tn_f64.argtypes = [
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
            ctypes.c_int]
        L.oracle_fa_fwd_f32.restype = None
        L.oracle_fa_fwd_f32.argtypes = [
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_void_p, i64p, ctypes.c_void_p, i64p, ctypes.c_void_p, i64p,
            ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        L.oracle_compare.restype = ctypes.c_int64
        L.oracle_compare.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                     ctypes.c_double, ctypes.c_double, ctypes.c_void_p]
        _lib = L
    return _lib


def num_threads():
    return int(lib().oracle_num_threads())


def use_all_cores():
    """Use every core this process may run on, whatever OMP_NUM_THREADS says (torchrun
    exports OMP_NUM_THREADS=1).  Returns the thread count now in effect."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_num_threads(n)
    return num_threads()


# Bit-pattern helpers and the seeded input generators live with the package (numpy only, no
# oracle code involved) so that the benchmark's GPU arm can draw its inputs without loading
# anything from this directory; they are re-exported here for the tests.
import sys as _sys

_ROOT = os.path.dirname(_HERE)
if _ROOT not in _sys.path:
    _sys.path.insert(0, _ROOT)
from sm120_dl_b200.synthetic import (bf16_bits_from_f32, f16_bits, f32_from_bf16_bits,  # noqa: E402,F401
                                     make_fa_inputs, make_gemm_inputs)


# ------------------------------------------------------------------------ C++ oracle
def gemm_f64(a_bits, b_bits, row_begin=0, row_count=None):
    """a_bits [M,K], b_bits [N,K] uint16 bf16 patterns -> float64 [row_count, N]."""
    a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    M, K = a_bits.shape
    N, K2 = b_bits.shape
    assert K == K2
    if row_count is None:
        row_count = M - row_begin
    assert 0 <= row_begin and row_begin + row_count <= M
    out = np.empty((row_count, N), dtype=np.float64)
    lib().oracle_gemm_bf16_tn_f64(M, N, K, a_bits.ctypes.data, K, b_bits.ctypes.data, K,
                                  out.ctypes.data, N, row_begin, row_count)
    return out


def _strides3(t):
    s = [st // t.itemsize for st in t.strides]
    assert s[3] == 1, "dim stride must be 1"
    return (ctypes.c_int64 * 3)(s[0], s[1], s[2])


def attention_f32(q_bits, k_bits, v_bits, causal=False, scale=None, rows=None):
    """q/k/v [B,S,H,D] uint16 fp16 patterns -> float32 [B, n_rows, H, D]."""
    B, Sq, H, D = q_bits.shape
    Sk = k_bits.shape[1]
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    if rows is not None:
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        n_rows = len(rows)
        rows_ptr = rows.ctypes.data
    else:
        n_rows = Sq
        rows_ptr = None
    out = np.empty((B, n_rows, H, D), dtype=np.float32)
    lib().oracle_fa_fwd_f32(B, Sq, Sk, H, D, q_bits.ctypes.data, _strides3(q_bits),
                            k_bits.ctypes.data, _strides3(k_bits), v_bits.ctypes.data,
                            _strides3(v_bits), float(scale), int(bool(causal)), rows_ptr,
                            n_rows, out.ctypes.data)
    return out


def compare(got, ref, abs_tol, rel_tol):
    """Reference-style comparison.  Returns a dict of error statistics."""
    got = np.ascontiguousarray(got, dtype=np.float64).ravel()
    ref = np.ascontiguousarray(ref, dtype=np.float64).ravel()
    assert got.shape == ref.shape
    stats = np.zeros(6, dtype=np.float64)
    bad = lib().oracle_compare(got.ctypes.data, ref.ctypes.data, got.size, float(abs_tol),
                               float(rel_tol), stats.ctypes.data)
    return {
        "mismatches": int(bad), "count": int(got.size), "passed": bad == 0,
        "max_abs": float(stats[0]), "max_rel": float(stats[1]), "first_bad": int(stats[2]),
        "max_ref": float(stats[3]), "rms_ref": float(stats[4]),
        # |diff| / max(|ref_i|, rms(ref)): relative error that stays bounded where ref ~ 0
        "max_rel_bounded": float(stats[5]),
    }


# --------------------------------------------------------------------- numpy restatement
def gemm_numpy(a_bits, b_bits):
    a = f32_from_bf16_bits(a_bits).astype(np.float64)
    b = f32_from_bf16_bits(b_bits).astype(np.float64)
    return a @ b.T


def attention_numpy(q_bits, k_bits, v_bits, causal=False, scale=None):
    q = q_bits.view(np.float16).astype(np.float64)
    k = k_bits.view(np.float16).astype(np.float64)
    v = v_bits.view(np.float16).astype(np.float64)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    s = np.einsum("bihd,bjhd->bhij", q, k) * scale
    if causal:
        i = np.arange(Sq)[:, None]
        j = np.arange(Sk)[None, :]
        s = np.where(i < j, -np.inf, s)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhij,bjhd->bihd", p, v)
