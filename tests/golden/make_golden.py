"""Generates the fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py

The reference (HugeOrca/sm120-dl) stores no expected outputs for either hot path -- its
checks compare against cuBLAS and flash-attn on the GPU at run time -- so these fixtures
pin the CPU oracle against INDEPENDENT CPU implementations instead:

  gemm_*.npz       torch.matmul in float64 on the CPU (operands exactly representable)
  attention_*.npz  torch.nn.functional.scaled_dot_product_attention in float64 on the CPU

Inputs come from the oracle's seeded generators (numpy PCG64), so a fixture holds only the
seed, the shape and the expected output.
"""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

GEMM_CASES = [
    # name, M, N, K, seed, dist
    ("gemm_u1_96x80x64", 96, 80, 64, 0, "uniform1"),
    ("gemm_n_128x256x192", 128, 256, 192, 1, "normal_over_sqrt_k"),
    ("gemm_u01_64x64x1024", 64, 64, 1024, 7, "uniform01"),
]
FA_CASES = [
    # name, B, S, H, D, seed, causal
    ("attention_b2_s96_h3_d64", 2, 96, 3, 64, 3, False),
    ("attention_b1_s160_h2_d128", 1, 160, 2, 128, 2, False),
    ("attention_b1_s128_h2_d128_causal", 1, 128, 2, 128, 5, True),
    ("attention_b2_s65_h1_d64_causal", 2, 65, 1, 64, 11, True),
]


def main():
    torch.set_num_threads(4)
    for name, M, N, K, seed, dist in GEMM_CASES:
        a, b = oracle.make_gemm_inputs(M, N, K, seed, dist)
        ta = torch.from_numpy(oracle.f32_from_bf16_bits(a)).double()
        tb = torch.from_numpy(oracle.f32_from_bf16_bits(b)).double()
        c = (ta @ tb.T).numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), shape=np.array([M, N, K]), seed=seed,
                            dist=dist, expected=c)
    for name, B, S, H, D, seed, causal in FA_CASES:
        q, k, v = oracle.make_fa_inputs(B, S, H, D, seed)
        tq, tk, tv = (torch.from_numpy(x.view(np.float16)).double().permute(0, 2, 1, 3) for x in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(tq, tk, tv, is_causal=causal)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), shape=np.array([B, S, H, D]), seed=seed,
                            causal=causal, expected=o.permute(0, 2, 1, 3).contiguous().numpy().astype(np.float32))
    print("wrote", len(GEMM_CASES) + len(FA_CASES), "fixtures to", HERE)


if __name__ == "__main__":
    main()
