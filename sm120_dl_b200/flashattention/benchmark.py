#!/usr/bin/env python3
"""Timing of the flashatten_v3_sm120 configs against a library attention.

Same command line, protocol and output as the reference script
(flashattention/v3_mMnNkN/benchmark.py of HugeOrca/sm120-dl): --config, --causal
(both/true/false), --warmup (5), --iterations (20), --case SEQ HEAD_DIM HEADS BATCH, --all;
CUDA events around back-to-back calls (benchmark.py:73-85); inputs randn * 0.5 seeded with
20260617 + sum of the shape (benchmark.py:63-70); per-config lines
"<case> <config> <elements/s> <ms>" and one summary line per case, also written to
benchmark.txt beside this file.  The reference's throughput unit is output elements per
second, B*H*S*D / t (benchmark.py:88-90); this script appends the attention FLOP rate,
4*B*H*S^2*D / t (halved when causal), to the summary line.

Comparator: flash_attn.flash_attn_func when importable, else torch SDPA in fp16.
"""

import argparse
import math
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "pybind" / "build"))
import flashatten_v3_sm120 as fa  # noqa: E402

from verify import SHAPES, as_bool, library_attention, _flash_attn_func  # noqa: E402

OUTPUT = Path(__file__).resolve().parent / "benchmark.txt"
OFFICIAL_NAME = "flash_attn_func" if _flash_attn_func is not None else "torch_sdpa"


def make_inputs(shape, causal):
    seq_len, head_dim, head_num, batch = shape
    torch.manual_seed(20260617 + seq_len + head_dim + head_num + batch + int(causal))
    q = (torch.randn(batch, seq_len, head_num, head_dim, device="cuda", dtype=torch.float16) * 0.5).contiguous()
    k = (torch.randn_like(q) * 0.5).contiguous()
    v = (torch.randn_like(q) * 0.5).contiguous()
    return q, k, v


def time_call(fn, warmup, iterations):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iterations):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iterations


def elements_per_second(shape, ms):
    seq_len, head_dim, head_num, batch = shape
    return batch * head_num * seq_len * head_dim / (ms * 1.0e-3)


def tflops(shape, causal, ms):
    seq_len, head_dim, head_num, batch = shape
    flop = 4.0 * batch * head_num * seq_len * seq_len * head_dim * (0.5 if causal else 1.0)
    return flop / (ms * 1.0e-3) / 1.0e12


def si(value):
    for suffix in ("", "K", "M", "G", "T"):
        if abs(value) < 1000.0:
            return f"{value:.3f}{suffix}"
        value /= 1000.0
    return f"{value:.3f}P"


def label(shape, causal):
    seq_len, head_dim, head_num, batch = shape
    return f"b{batch}_hn{head_num}_seq{seq_len}_hd{head_dim}_casual{int(causal)}"


def benchmark_shape(configs, shape, causal, warmup, iterations):
    seq_len, head_dim, _, _ = shape
    q, k, v = make_inputs(shape, causal)
    rows = []
    with torch.no_grad():
        for name, cfg_dim, block_m, block_n, _, _, _ in configs:
            if cfg_dim != head_dim or seq_len % block_m or seq_len % block_n:
                continue
            ms = time_call(lambda: fa.fwd_config(name, q, k, v, causal), warmup, iterations)
            rows.append((name, elements_per_second(shape, ms), ms))
        lib_ms = time_call(lambda: library_attention(q, k, v, causal), warmup, iterations)
    tag = label(shape, causal)
    for name, rate, ms in sorted(rows, key=lambda r: r[1], reverse=True):
        print(f"{tag} {name} {si(rate)} {ms:.6f}", flush=True)
    del q, k, v
    torch.cuda.empty_cache()
    if not rows:
        return None
    best = max(rows, key=lambda r: r[1])
    lib_rate = elements_per_second(shape, lib_ms)
    return (f"{tag} {best[0]}: {si(best[1])} {best[2]:.6f} {OFFICIAL_NAME}: {si(lib_rate)} {lib_ms:.6f} "
            f"custom/official:{best[1] / lib_rate * 100.0:.2f}% "
            f"tflops:{tflops(shape, causal, best[2]):.1f} official_tflops:{tflops(shape, causal, lib_ms):.1f}")


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--config", help="benchmark one config by exact name")
    ap.add_argument("--causal", help="both, true, or false")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--case", nargs=4, type=int, metavar=("SEQ_LEN", "HEAD_DIM", "HEAD_NUM", "BATCH"))
    ap.add_argument("--all", action="store_true", help="benchmark all shapes of verify.py")
    args = ap.parse_args()
    if args.warmup < 0:
        raise SystemExit("--warmup must be non-negative")
    if args.iterations <= 0:
        raise SystemExit("--iterations must be positive")

    configs = fa.configs()
    if args.config:
        configs = [c for c in configs if c[0] == args.config]
        if not configs:
            raise SystemExit(f"unknown --config '{args.config}'. available: {', '.join(c[0] for c in fa.configs())}")
    shapes = SHAPES if args.all or not args.case else [tuple(args.case)]
    if args.causal is None:
        causal_modes = (False, True) if args.all else (False,)
    elif args.causal == "both":
        causal_modes = (False, True)
    else:
        causal_modes = (as_bool(args.causal),)

    lines = []
    for shape in shapes:
        for causal in causal_modes:
            line = benchmark_shape(configs, shape, causal, args.warmup, args.iterations)
            if line:
                print(line, flush=True)
                lines.append(line)
    OUTPUT.write_text("\n".join(lines) + ("\n" if lines else ""), encoding="utf-8")


if __name__ == "__main__":
    main()
