#!/usr/bin/env python3
"""One attention-forward launch between cudaProfilerStart/Stop, for Nsight Compute.

Same command line as the reference script (flashattention/v3_mMnNkN/test_compute_rate.py
of HugeOrca/sm120-dl: --func, --seq-len, --head-num, --batch, --causal, --warmup, --sleep,
--list, --list-names).  Typical use:

    ncu --profile-from-start off --clock-control none -c 1 \\
        --metrics sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed,dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum \\
        python test_compute_rate.py --func <config> --seq-len 4096 --head-num 32 --batch 1 --sleep 0
"""

import argparse
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "pybind" / "build"))
import flashatten_v3_sm120 as fa  # noqa: E402


def as_bool(text):
    if text in ("1", "true", "True", "yes", "y"):
        return True
    if text in ("0", "false", "False", "no", "n"):
        return False
    raise argparse.ArgumentTypeError(f"invalid bool: {text}")


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--func", help="flash_fwd config name (see --list)")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--head-num", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--causal", type=as_bool, default=False)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--sleep", type=float, default=10.0)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--list-names", action="store_true")
    args = ap.parse_args()

    table = {c[0]: c for c in fa.configs()}
    if args.list or args.list_names:
        for name, hd, bm, bn, nwarps, stage, smem in table.values():
            print(name if args.list_names else f"{name} hd={hd} bm={bm} bn={bn} nwarps={nwarps} stage={stage} smem={smem}")
        return 0
    if not args.func:
        ap.error("--func is required unless --list or --list-names is used")
    if args.func not in table:
        raise SystemExit(f"unknown --func '{args.func}'. available: {', '.join(table)}")
    if min(args.seq_len, args.head_num, args.batch) <= 0 or args.warmup < 0 or args.sleep < 0:
        ap.error("sizes must be positive, --warmup and --sleep non-negative")
    _, head_dim, block_m, block_n, _, _, _ = table[args.func]
    if args.seq_len % block_m or args.seq_len % block_n:
        raise SystemExit(f"{args.func} expects seq_len to be a multiple of {block_m} and {block_n}, got {args.seq_len}")

    cudart = torch.cuda.cudart()
    with torch.no_grad():
        torch.manual_seed(20260629 + args.seq_len + head_dim + args.head_num + args.batch + int(args.causal))
        q = torch.randn(args.batch, args.seq_len, args.head_num, head_dim, device="cuda", dtype=torch.float16) * 0.5
        k = torch.randn_like(q) * 0.5
        v = torch.randn_like(q) * 0.5
        for _ in range(args.warmup):
            fa.fwd_config(args.func, q, k, v, args.causal)
        torch.cuda.synchronize()
        print(f"PROFILE func={args.func} seq_len={args.seq_len} head_dim={head_dim} head_num={args.head_num} "
              f"batch={args.batch} causal={int(args.causal)}", flush=True)
        cudart.cudaProfilerStart()
        try:
            out = fa.fwd_config(args.func, q, k, v, args.causal)
            torch.cuda.synchronize()
        finally:
            cudart.cudaProfilerStop()
        print(f"DONE func={args.func} output_shape={tuple(out.shape)}", flush=True)
    if args.sleep > 0:
        time.sleep(args.sleep)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
