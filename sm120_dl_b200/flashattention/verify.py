#!/usr/bin/env python3
"""Parity check of the flashatten_v3_sm120 module against a library attention.

Same command line, shape list, inputs, tolerance and result lines as the reference script
(flashattention/v3_mMnNkN/verify.py of HugeOrca/sm120-dl):

    verify.py                              the 18 built-in shapes x {non-causal, causal} through fwd()
    verify.py --all                        every config x head count x causal once, through fwd_config()
    verify.py --case SEQ HEAD_DIM HEADS BATCH CAUSAL

The comparator is flash_attn.flash_attn_func when that package imports (the reference's
comparator, verify.py:8,129), otherwise torch's scaled_dot_product_attention in fp16.
Inputs: torch.manual_seed(20260614 + sum of the shape), randn * 0.5 (verify.py:56-61).
Pass rule: |got - ref| <= 0.075 + 0.075 |ref|, no non-finite value (verify.py:64-80).
--tight additionally requires max |got - fp32 reference| <= 2e-3.
"""

import argparse
import math
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "pybind" / "build"))
import flashatten_v3_sm120 as fa  # noqa: E402

try:
    from flash_attn import flash_attn_func as _flash_attn_func
except Exception:  # the comparator package is optional on a B200 box
    _flash_attn_func = None

ATOL = 7.5e-2
RTOL = 7.5e-2
TIGHT_ABS = 2.0e-3
HEAD_NUMS = (1, 4, 8, 16, 32, 64, 80)
# seq_len, head_dim, head_num, batch
SHAPES = [
    (64, 64, 1, 1), (128, 64, 1, 1), (128, 64, 1, 2), (192, 64, 1, 1), (128, 64, 4, 1), (192, 64, 4, 1),
    (256, 64, 8, 2), (128, 128, 4, 1), (128, 128, 4, 2), (256, 128, 4, 1), (2048, 64, 16, 1),
    (4096, 128, 32, 1), (8192, 128, 32, 1), (16384, 128, 32, 1), (2048, 64, 32, 8), (4096, 128, 64, 2),
    (4096, 128, 64, 8), (8192, 128, 80, 4),
]


def as_bool(text):
    if text in ("1", "true", "True", "yes", "y"):
        return True
    if text in ("0", "false", "False", "no", "n"):
        return False
    raise argparse.ArgumentTypeError(f"invalid bool: {text}")


def make_inputs(seq_len, head_dim, head_num, batch, causal):
    torch.manual_seed(20260614 + seq_len + head_dim + head_num + batch + int(causal))
    q = (torch.randn(batch, seq_len, head_num, head_dim, device="cuda", dtype=torch.float16) * 0.5).contiguous()
    k = (torch.randn_like(q) * 0.5).contiguous()
    v = (torch.randn_like(q) * 0.5).contiguous()
    return q, k, v


def library_attention(q, k, v, causal, dtype=None):
    """[B,S,H,D] in, [B,S,H,D] out."""
    if _flash_attn_func is not None and dtype is None:
        return _flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=1.0 / math.sqrt(q.size(3)), causal=causal)
    qq, kk, vv = (t.transpose(1, 2) if dtype is None else t.transpose(1, 2).to(dtype) for t in (q, k, v))
    out = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=causal)
    return out.transpose(1, 2)


def compare(got, ref):
    diff = (got.float() - ref.float()).abs()
    bad = (diff > ref.float().abs() * RTOL + ATOL) | ~torch.isfinite(got) | ~torch.isfinite(ref)
    diff = torch.nan_to_num(diff, nan=float("inf"), posinf=float("inf"), neginf=float("inf"))
    max_abs = diff.max().item()
    max_rel = torch.nan_to_num(diff / ref.float().abs().clamp_min(1.0e-6), nan=float("inf")).max().item()
    return (not bool(bad.any())), max_abs, max_rel, int(bad.sum().item()), got.numel()


def case_name(seq_len, head_dim, head_num, batch, causal):
    return f"b{batch}_hn{head_num}_seq{seq_len}_hd{head_dim}_casual{int(causal)}"


def report(status, shape, causal, stats, config=None):
    max_abs, max_rel, bad, total = stats
    prefix = f"{status} {case_name(*shape, causal)}" + (f" {config}" if config else "")
    print(f"{prefix} max_abs={max_abs:.6g} max_rel={max_rel:.6g} mismatches={bad}/{total}", flush=True)


def run_case(shape, causal, config=None, tight=False):
    seq_len, head_dim, head_num, batch = shape
    with torch.no_grad():
        q, k, v = make_inputs(seq_len, head_dim, head_num, batch, causal)
        try:
            got = fa.fwd_config(config, q, k, v, causal) if config else fa.fwd(q, k, v, causal)
        except RuntimeError as exc:
            print(f"FAIL {case_name(*shape, causal)}" + (f" {config}" if config else "") + f" error={exc}", flush=True)
            return False
        ref = library_attention(q, k, v, causal)
        torch.cuda.synchronize()
        ok, *stats = compare(got, ref)
        if tight and ok and batch * head_num * seq_len * seq_len <= 2 ** 31:
            exact = library_attention(q, k, v, causal, dtype=torch.float32)
            err = (got.float() - exact).abs().max().item()
            if not err <= TIGHT_ABS:
                print(f"FAIL {case_name(*shape, causal)} fp32 reference max_abs={err:.6g} > {TIGHT_ABS}", flush=True)
                ok = False
    report("PASS" if ok else "FAIL", shape, causal, stats, config)
    del q, k, v, got, ref
    torch.cuda.empty_cache()
    return ok


def run_all_configs(tight):
    ok, passed, total = True, 0, 0
    configs = fa.configs()
    for name, head_dim, block_m, block_n, _, _, _ in configs:
        seq_len = math.lcm(block_m, block_n)
        for head_num in HEAD_NUMS:
            for causal in (False, True):
                good = run_case((seq_len, head_dim, head_num, 1), causal, config=name, tight=tight)
                ok &= good
                passed += int(good)
                total += 1
    print(f"SUMMARY kernel_templates passed={passed}/{total} configs={len(configs)} head_nums={len(HEAD_NUMS)} "
          f"causals=2 resource_skips=0", flush=True)
    return ok


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--case", nargs=5, metavar=("SEQ_LEN", "HEAD_DIM", "HEAD_NUM", "BATCH", "CAUSAL"))
    ap.add_argument("--all", "--all-configs", dest="all_configs", action="store_true",
                    help="verify every config x head count x causal")
    ap.add_argument("--tight", action="store_true", help="also require max abs error <= 2e-3 vs an fp32 reference")
    args = ap.parse_args()
    if args.case:
        if args.all_configs:
            ap.error("--all cannot be combined with --case")
        shape = tuple(int(x) for x in args.case[:4])
        return 0 if run_case(shape, as_bool(args.case[4]), tight=args.tight) else 1
    if args.all_configs:
        return 0 if run_all_configs(args.tight) else 1
    ok = True
    for shape in SHAPES:
        for causal in (False, True):
            ok &= run_case(shape, causal, tight=args.tight)
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
