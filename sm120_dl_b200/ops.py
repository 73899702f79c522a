"""Torch-facing operators over the C ABI: the calls a Python user makes.

  gemm_bf16_tn(a, b)            C = A @ B.T  (a [M,K], b [N,K] bf16 CUDA tensors)
  flash_attn_fwd(q, k, v, ...)  O = softmax(Q K^T / sqrt(D)) V on [B,S,H,D] fp16 CUDA tensors

Torch is used for device memory and streams only; the arithmetic happens in
libb200dl.so.  Tensors may be views (column slabs, head slices): leading dimensions and
strides are passed through, which is what the sharded multi-GPU path relies on.
"""

import ctypes
import math

import torch

from . import capi


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_matrix(t, name, dtype):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must use {dtype}")
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit stride along the last dimension")


def gemm_config_index(name_or_index, M, N, K):
    L = capi.lib()
    if name_or_index is None:
        idx = L.b200_gemm_default_config(M, N, K)
        if idx < 0:
            raise capi.B200Error(-2, f"no built GEMM config divides the shape {M}x{N}x{K}")
        return idx
    if isinstance(name_or_index, int):
        return name_or_index
    idx = L.b200_gemm_find_config(name_or_index.encode())
    if idx < 0:
        raise ValueError(f"unknown GEMM config: {name_or_index}")
    return idx


def gemm_bf16_tn(a, b, out=None, config=None):
    """C[M,N] = A[M,K] @ B[N,K]^T, bf16 in / fp32 accumulate / bf16 out, on the current
    stream of a's device.  `out` may be a column slab of a wider matrix."""
    _check_matrix(a, "a", torch.bfloat16)
    _check_matrix(b, "b", torch.bfloat16)
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if b.device != a.device:
        raise ValueError("a and b must be on the same device")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    else:
        _check_matrix(out, "out", torch.bfloat16)
        if tuple(out.shape) != (M, N) or out.device != a.device:
            raise ValueError("out has the wrong shape or device")
    idx = gemm_config_index(config, M, N, K)
    with torch.cuda.device(a.device):
        capi.check(capi.lib().b200_gemm_bf16_tn(
            idx, M, N, K, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
            out.data_ptr(), out.stride(0), _stream_ptr(a.device)))
    return out


def gemm_f16_tn(a, b, out=None, config=None):
    """C = A @ B^T for fp16 operands and output (fp32 accumulation)."""
    _check_matrix(a, "a", torch.float16)
    _check_matrix(b, "b", torch.float16)
    M, K = a.shape
    N, K2 = b.shape
    if K != K2 or b.device != a.device:
        raise ValueError("a [M,K] and b [N,K] must share K and the device")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=a.device)
    else:
        _check_matrix(out, "out", torch.float16)
        if tuple(out.shape) != (M, N) or out.device != a.device:
            raise ValueError("out has the wrong shape or device")
    idx = gemm_config_index(config, M, N, K)
    with torch.cuda.device(a.device):
        capi.check(capi.lib().b200_gemm_f16_tn(
            idx, M, N, K, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
            out.data_ptr(), out.stride(0), _stream_ptr(a.device)))
    return out


def gemm_bf16_tn_scatter(a, b, outs, config=None):
    """C = A @ B^T written to every tensor in `outs` (1..8 [M,N] windows with one common
    leading dimension; they may alias other GPUs' memory, e.g. symmetric-memory buffers)."""
    _check_matrix(a, "a", torch.bfloat16)
    _check_matrix(b, "b", torch.bfloat16)
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if not 1 <= len(outs) <= 8:
        raise ValueError("between 1 and 8 destinations are supported")
    for t in outs:
        _check_matrix(t, "out", torch.bfloat16)
        if tuple(t.shape) != (M, N) or t.stride(0) != outs[0].stride(0):
            raise ValueError("every destination must be an [M,N] window with the same leading dimension")
    idx = gemm_config_index(config, M, N, K)
    ptrs = (ctypes.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
    with torch.cuda.device(a.device):
        capi.check(capi.lib().b200_gemm_bf16_tn_scatter(
            idx, M, N, K, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), ptrs, len(outs),
            outs[0].stride(0), _stream_ptr(a.device)))
    return outs


def _check_bshd(t, name):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.float16:
        raise ValueError(f"{name} must use torch.float16")
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError(f"{name} must have shape [batch, seq_len, head_num, head_dim] with unit stride along head_dim")


def _strides3(t):
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def fa_config_index(name_or_index, head_dim):
    L = capi.lib()
    if name_or_index is None:
        idx = L.b200_fa_default_config(head_dim)
        if idx < 0:
            raise capi.B200Error(-2, f"no flash_fwd config was built for head_dim={head_dim}")
        return idx
    if isinstance(name_or_index, int):
        return name_or_index
    idx = L.b200_fa_find_config(name_or_index.encode())
    if idx < 0:
        raise ValueError(f"unknown flash_fwd config: {name_or_index}")
    return idx


def flash_attn_fwd(q, k, v, causal=False, softmax_scale=None, out=None, config=None):
    """Attention forward on [B,S,H,D] fp16 tensors (views with strides are accepted);
    returns a new contiguous tensor unless `out` is given."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_bshd(t, n)
    B, Sq, H, D = q.shape
    if k.shape != v.shape or k.shape[0] != B or k.shape[2] != H or k.shape[3] != D:
        raise ValueError("k and v must match q in batch, heads and head_dim, and each other in seq_len")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must be on the same device")
    Sk = k.shape[1]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=torch.float16, device=q.device)
    else:
        _check_bshd(out, "out")
        if tuple(out.shape) != (B, Sq, H, D) or out.device != q.device:
            raise ValueError("out has the wrong shape or device")
    idx = fa_config_index(config, D)
    with torch.cuda.device(q.device):
        capi.check(capi.lib().b200_fa_fwd_fp16(
            idx, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Sq, Sk, H, D,
            _strides3(q), _strides3(k), _strides3(v), _strides3(out), float(softmax_scale),
            int(bool(causal)), _stream_ptr(q.device)))
    return out


def flash_attn_fwd_scatter(q, k, v, outs, causal=False, softmax_scale=None, config=None):
    """Attention forward written to every tensor in `outs` (1..8 [B,S,H,D] windows with
    identical strides; they may alias other GPUs' memory)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_bshd(t, n)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    if not 1 <= len(outs) <= 8:
        raise ValueError("between 1 and 8 destinations are supported")
    for t in outs:
        _check_bshd(t, "out")
        if tuple(t.shape) != (B, Sq, H, D) or t.stride() != outs[0].stride():
            raise ValueError("every destination must be a [B,S,H,D] window with the same strides")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    idx = fa_config_index(config, D)
    ptrs = (ctypes.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
    with torch.cuda.device(q.device):
        capi.check(capi.lib().b200_fa_fwd_fp16_scatter(
            idx, q.data_ptr(), k.data_ptr(), v.data_ptr(), ptrs, len(outs), B, Sq, Sk, H, D,
            _strides3(q), _strides3(k), _strides3(v), _strides3(outs[0]), float(softmax_scale),
            int(bool(causal)), _stream_ptr(q.device)))
    return outs
