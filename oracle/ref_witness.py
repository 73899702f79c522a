"""ctypes face of oracle/_ref/libsm120ref.so (the reference project's kernels rebuilt for
sm_100a by oracle/build_ref.py).  TEST INFRASTRUCTURE ONLY: used by the parity tests as a
same-box witness and, run as a script, to time those kernels for the comparison tables.

    python oracle/ref_witness.py          # times the reference kernels on the benchmark shapes
"""

import ctypes
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libsm120ref.so")

GEMM_CONFIGS = {0: "bf16_bm128_bn64_bk64_s3_cwg2_wm2_wn4_bsw8", 1: "bf16_bm128_bn128_bk64_s2_cwg2_wm2_wn4_bsw8"}
FA_CONFIGS = {128: "hd128_bm128_bn64_wm8_wn1_s2", 64: "hd64_bm128_bn32_wm8_wn1_s2"}
FA_HEADS = {128: (4, 32), 64: (4, 32)}

_lib = None


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(LIB_PATH)
        vp = ctypes.c_void_p
        L.ref_gemm_bf16_tn.restype = ctypes.c_int
        L.ref_gemm_bf16_tn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp, vp, vp]
        for d, heads in FA_HEADS.items():
            for h in heads:
                fn = getattr(L, f"ref_fa_fwd_fp16_d{d}_h{h}")
                fn.restype = ctypes.c_int
                fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp, vp, vp, ctypes.c_float, vp]
        _lib = L
    return _lib


def gemm(which, a, b, c, stream=None):
    """C = A @ B^T with the reference's gemm_tn (contiguous bf16 torch CUDA tensors)."""
    M, K = a.shape
    N = b.shape[0]
    rc = lib().ref_gemm_bf16_tn(which, M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)
    if rc != 0:
        raise RuntimeError(f"reference gemm_tn config {which} refused {M}x{N}x{K} (rc {rc})")
    return c


def attention(q, k, v, o, causal, stream=None):
    """The reference's flash_fwd on contiguous [B,S,H,D] fp16 torch CUDA tensors."""
    B, S, H, D = q.shape
    if D not in FA_HEADS or H not in FA_HEADS[D]:
        raise RuntimeError(f"reference flash_fwd was not instantiated for head_dim {D}, heads {H}")
    fn = getattr(lib(), f"ref_fa_fwd_fp16_d{D}_h{H}")
    rc = fn(int(bool(causal)), B, S, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 1.0 / D ** 0.5, stream)
    if rc != 0:
        raise RuntimeError(f"reference flash_fwd refused B{B} S{S} H{H} D{D} (rc {rc})")
    return o


def _time(fn, iters, torch):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    import torch
    if not available():
        print("oracle/_ref/libsm120ref.so is not built (python oracle/build_ref.py)")
        return 1
    dev = torch.device("cuda:0")
    print("| kernel (reference source, rebuilt for sm_100a) | shape | ms | TFLOP/s |")
    print("|---|---|---:|---:|")
    for (M, N, K) in ((8192, 8192, 8192), (16384, 4096, 4096)):
        a = (torch.randn(M, K, device=dev) / K ** 0.5).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        for which, name in GEMM_CONFIGS.items():
            ms = _time(lambda: gemm(which, a, b, c), 10, torch)
            print(f"| gemm_tn {name} | {M}x{N}x{K} | {ms:.4f} | {2.0 * M * N * K / ms / 1e9:.1f} |")
    for (B, H, S, D) in ((4, 32, 4096, 128), (16, 32, 2048, 64)):
        q, k, v = (torch.randn(B, S, H, D, device=dev).to(torch.float16) for _ in range(3))
        o = torch.empty_like(q)
        for causal in (False, True):
            ms = _time(lambda: attention(q, k, v, o, causal), 10, torch)
            fl = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
            print(f"| flash_fwd {FA_CONFIGS[D]} causal={int(causal)} | B{B} H{H} S{S} D{D} | {ms:.4f} | {fl / ms / 1e9:.1f} |")
    return 0


if __name__ == "__main__":
    sys.exit(main())
