#!/usr/bin/env python3
"""Run one attention-forward case with one kernel config and print its time.

Command line and output lines of the reference's single-case runner
(flashattention/v3_mMnNkN/test.py:100-141): without arguments the built configs are
listed; with `--config` and `--func` one case runs once between two CUDA events.

    python test.py
    python test.py --config b4_hn32_seq4096_hd128_casual0 --func hd128_bm64_bn64_tq128x2_tk128_s5_e0
    python test.py --config 4096 128 32 4 0 --func ...       # SEQ_LEN HEAD_DIM HEAD_NUM BATCH CAUSAL

Inputs: N(0,1)*0.5 fp16 from torch.manual_seed(20260623 + seq + dim + heads + batch + causal)
(test.py:88-93).  `throughput` is batch*heads*seq*dim elements per second, the reference's
unit (test.py:131); tflops is added for the B200 reports.
"""
import argparse
import os
import re
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "pybind", "build"))
import flashatten_v3_sm120  # noqa: E402

LABEL = re.compile(r"^b(\d+)_hn(\d+)_seq(\d+)_hd(\d+)_(?:casual|causal)([01])$")
TRUE, FALSE = ("1", "true", "True", "yes", "y"), ("0", "false", "False", "no", "n")


def parse_case(values):
    """-> (seq_len, head_dim, head_num, batch, causal) from a label, a comma list or 5 words."""
    if len(values) == 1:
        m = LABEL.match(values[0])
        if m:
            batch, heads, seq, dim, causal = (int(x) for x in m.groups())
            return seq, dim, heads, batch, bool(causal)
        if "," in values[0]:
            values = [v.strip() for v in values[0].split(",") if v.strip()]
    if len(values) != 5 or values[4] not in TRUE + FALSE:
        raise SystemExit("--config expects either b<B>_hn<H>_seq<S>_hd<D>_casual<0|1> "
                         "or: SEQ_LEN HEAD_DIM HEAD_NUM BATCH CAUSAL")
    seq, dim, heads, batch = (int(v) for v in values[:4])
    return seq, dim, heads, batch, values[4] in TRUE


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--config", nargs="+", metavar="INPUT")
    ap.add_argument("--func", help="kernel config name")
    args = ap.parse_args()
    configs = flashatten_v3_sm120.configs()
    if args.config is None and args.func is None:
        for name, head_dim, block_m, block_n, nwarps, stage, smem in configs:
            print(f"{name} hd={head_dim} bm={block_m} bn={block_n} nwarps={nwarps} stage={stage} smem={smem}")
        return 0
    if args.config is None or args.func is None:
        ap.error("--config and --func must be provided together")
    seq, dim, heads, batch, causal = parse_case(args.config)
    chosen = [c for c in configs if c[0] == args.func]
    if not chosen:
        raise SystemExit(f"unknown --func '{args.func}'. available: " + ", ".join(c[0] for c in configs))
    name, cfg_dim, block_m, block_n = chosen[0][:4]
    if dim != cfg_dim:
        raise SystemExit(f"{name} expects head_dim={cfg_dim}, got {dim}")
    for what, block in (("block_m", block_m), ("block_n", block_n)):
        if seq % block:
            raise SystemExit(f"{name} expects seq_len to be a multiple of {what}={block}, got {seq}")

    label = f"b{batch}_hn{heads}_seq{seq}_hd{dim}_casual{int(causal)}"
    print(f"RUN {label} func={name}", flush=True)
    with torch.no_grad():
        torch.manual_seed(20260623 + seq + dim + heads + batch + int(causal))
        q = (torch.randn(batch, seq, heads, dim, device="cuda", dtype=torch.float16) * 0.5).contiguous()
        k = (torch.randn_like(q) * 0.5).contiguous()
        v = (torch.randn_like(q) * 0.5).contiguous()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = flashatten_v3_sm120.fwd_config(name, q, k, v, causal)
        stop.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    throughput = batch * heads * seq * dim / (ms * 1e-3)
    tflops = 4.0 * batch * heads * seq * seq * dim * (0.5 if causal else 1.0) / (ms * 1e-3) / 1e12
    print(f"DONE {label} func={name} elapsed_ms={ms:.6f} throughput={throughput / 1e9:.3f}G "
          f"tflops={tflops:.1f} output_shape={tuple(out.shape)}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
