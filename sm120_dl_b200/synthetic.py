"""Seeded synthetic operands of the benchmark configurations (numpy only).

The benchmark's inputs are not a dataset: they are random tensors of stated shape,
distribution and seed.  This module is the one place that draws them, so the kernels, the
CPU oracle and the committed fixtures all see the same bits.  Generator: numpy
PCG64(seed), float32 draws rounded to the storage type; A is drawn before B (the reference
harness fills A, B, C in that order, gemm/test.cpp:384-386) and q before k before v
(flashattention/v3_mMnNkN/verify.py:58-60).
"""

import numpy as np


def bf16_bits_from_f32(x):
    """float32 array -> uint16 bf16 bit patterns, round-to-nearest-even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def f32_from_bf16_bits(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def f16_bits(x):
    return np.ascontiguousarray(x, dtype=np.float16).view(np.uint16)


def make_gemm_inputs(M, N, K, seed, dist="normal_over_sqrt_k"):
    """Deterministic bf16 operands A [M,K], B [N,K] as uint16 bit patterns.

    dist: "uniform1" = uniform[-1,1) (the 512^3 configuration), "uniform01" =
    uniform[-0.1,0.1) (the reference harness), "normal_over_sqrt_k" = N(0,1)/sqrt(K).
    """
    rng = np.random.Generator(np.random.PCG64(seed))

    def draw(rows):
        if dist == "uniform1":
            x = rng.uniform(-1.0, 1.0, size=(rows, K)).astype(np.float32)
        elif dist == "uniform01":
            x = rng.uniform(-0.1, 0.1, size=(rows, K)).astype(np.float32)
        elif dist == "normal_over_sqrt_k":
            x = rng.standard_normal(size=(rows, K), dtype=np.float32) / np.float32(np.sqrt(K))
        else:
            raise ValueError(dist)
        return bf16_bits_from_f32(x)

    a = draw(M)
    b = draw(N)
    return a, b


def make_fa_inputs(B, S, H, D, seed, std=1.0):
    """Deterministic fp16 q, k, v [B,S,H,D] as uint16 bit patterns, N(0, std^2)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = []
    for _ in range(3):
        x = rng.standard_normal(size=(B, S, H, D), dtype=np.float32) * np.float32(std)
        out.append(f16_bits(x))
    return tuple(out)
