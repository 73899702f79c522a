#!/usr/bin/env python3
"""Fixed-size multi-GPU sweep: the same problems split over 1, 2, 4 or 8 GPUs (strong scaling).

    python -m sm120_dl_b200.sweep                                  # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m sm120_dl_b200.sweep [--out sweep.jsonl] [--iterations 20]

Workloads (seeded synthetic operands):
  BF16 GEMM M=16384, (N,K) in {(4096,4096), (14336,4096), (4096,14336)}, operands
  N(0,1)/sqrt(K), split by N-column blocks (A replicated, B row slab, C column slab);
  FP16 attention forward B=1 H=64 S=32768 D=128, N(0,1), split by heads.

Every rank times its shard with CUDA events (5 warm-up + `iterations` launches, the
reference harnesses' protocol); the job time is the maximum over ranks, the aggregate rate
is the WHOLE problem's flops divided by it.  A second figure includes the NCCL all-gather
that leaves the full output on every rank; a third uses the fused variant, where the kernel's
epilogue stores every tile into all ranks' output over NVLink and only a barrier follows.
One JSON line per (workload, world size) is printed by rank 0 and appended to --out; lines already present there are skipped, so an
interrupted sweep resumes where it stopped.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import capi, ops, sharded

GEMMS = [(16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336)]
ATTENTION = (1, 32768, 64, 128)  # B, S, H, D
SEED_GEMM, SEED_ATTENTION = 4, 5
WARMUP = 5


def timed(fn, iterations):
    for _ in range(WARMUP):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iterations):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iterations


def max_over_ranks(value, world, dev):
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_gemm(M, N, K, world, rank, dev, iterations):
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED_GEMM)
    a = (torch.randn(M, K, device=dev, generator=gen) / K ** 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev, generator=gen) / K ** 0.5).to(torch.bfloat16)
    n0, n1 = sharded.shard_bounds(N, world, rank, 256)
    slab = torch.empty((M, n1 - n0), dtype=torch.bfloat16, device=dev)
    cfg = ops.gemm_config_index(None, M, n1 - n0, K)
    compute_ms = timed(lambda: ops.gemm_bf16_tn(a, b[n0:n1], out=slab, config=cfg), iterations)
    gather_ms = None
    if world > 1:
        gather_ms = timed(lambda: sharded.gemm_column_shard(a, b, gather=True, granule=256, config=cfg), iterations)
        full, _ = sharded.gemm_column_shard(a, b, gather=True, granule=256, config=cfg)
        assert torch.equal(full[:, n0:n1].view(torch.int16), slab.view(torch.int16)), "gathered C differs from the shard"
    # the same all-gather pipelined over four row panels of A (gather of panel p under the GEMM of p+1)
    panel_ms = None
    if world > 1 and M % 4 == 0:
        panel_ms = timed(lambda: sharded.gemm_column_shard(a, b, gather=True, granule=256, config=cfg, panels=4),
                         iterations)
        piped, _ = sharded.gemm_column_shard(a, b, gather=True, granule=256, config=cfg, panels=4)
        assert torch.equal(piped.view(torch.int16), full.view(torch.int16)), "pipelined gather differs from the plain one"
        del piped
    fused_ms = None
    if world > 1:
        c_sym, handle = sharded.symmetric_empty((M, N), torch.bfloat16, dev)
        c_sym.fill_(float("nan"))
        handle.barrier()
        fused_ms = timed(lambda: sharded.gemm_column_shard_fused(a, b, c_sym, handle, granule=256, config=cfg),
                         iterations)
        torch.cuda.synchronize()
        handle.barrier()
        assert torch.equal(c_sym.view(torch.int16), full.view(torch.int16)), "fused gather differs from all-gather"
        del c_sym, handle
    assert capi.device_status() == 0
    flops = 2.0 * M * N * K
    return {"workload": f"gemm_bf16 M={M} N={N} K={K}", "flops": flops, "kernel_config": capi.gemm_configs()[cfg]["name"],
            "shard": f"columns [{n0},{n1}) of {N}", "compute_ms": compute_ms, "gather_ms": gather_ms,
            "panel_gather_ms": panel_ms, "fused_ms": fused_ms}


def run_attention(world, rank, dev, iterations):
    B, S, H, D = ATTENTION
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED_ATTENTION)
    q, k, v = (torch.randn(B, S, H, D, device=dev, generator=gen).to(torch.float16) for _ in range(3))
    h0, h1 = sharded.shard_bounds(H, world, rank)
    out = torch.empty((B, S, h1 - h0, D), dtype=torch.float16, device=dev)
    cfg = ops.fa_config_index(None, D)
    compute_ms = timed(lambda: ops.flash_attn_fwd(q[:, :, h0:h1], k[:, :, h0:h1], v[:, :, h0:h1], out=out, config=cfg),
                       iterations)
    gather_ms = None
    if world > 1:
        gather_ms = timed(lambda: sharded.attention_head_shard(q, k, v, gather=True, config=cfg), iterations)
        full, _ = sharded.attention_head_shard(q, k, v, gather=True, config=cfg)
        assert torch.equal(full[:, :, h0:h1].view(torch.int16), out.view(torch.int16)), "gathered O differs from the shard"
    fused_ms = None
    if world > 1:
        o_sym, handle = sharded.symmetric_empty((B, S, H, D), torch.float16, dev)
        o_sym.fill_(float("nan"))
        handle.barrier()
        fused_ms = timed(lambda: sharded.attention_head_shard_fused(q, k, v, o_sym, handle, config=cfg), iterations)
        torch.cuda.synchronize()
        handle.barrier()
        assert torch.equal(o_sym.view(torch.int16), full.view(torch.int16)), "fused gather differs from all-gather"
        del o_sym, handle
    assert capi.device_status() == 0
    flops = 4.0 * B * H * S * S * D
    return {"workload": f"fa_fwd_fp16 B={B} H={H} S={S} D={D}", "flops": flops,
            "kernel_config": capi.fa_configs()[cfg]["name"], "shard": f"heads [{h0},{h1}) of {H}",
            "compute_ms": compute_ms, "gather_ms": gather_ms, "fused_ms": fused_ms}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", default=None, help="JSON-lines file to append to (and resume from)")
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--skip-attention", action="store_true")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    done = set()
    if args.out and os.path.exists(args.out):
        with open(args.out) as f:
            for line in f:
                try:
                    rec = json.loads(line)
                    done.add((rec["workload"], rec["n_gpus"]))
                except (ValueError, KeyError):
                    pass

    jobs = [("gemm", shape) for shape in GEMMS] + ([] if args.skip_attention else [("attention", None)])
    for kind, shape in jobs:
        name = (f"gemm_bf16 M={shape[0]} N={shape[1]} K={shape[2]}" if kind == "gemm"
                else "fa_fwd_fp16 B=%d H=%d S=%d D=%d" % (ATTENTION[0], ATTENTION[2], ATTENTION[1], ATTENTION[3]))
        if (name, world) in done:
            continue
        rec = run_gemm(*shape, world, rank, dev, args.iterations) if kind == "gemm" else run_attention(
            world, rank, dev, args.iterations)
        compute_ms = max_over_ranks(rec["compute_ms"], world, dev)
        gather_ms = max_over_ranks(rec["gather_ms"], world, dev) if rec["gather_ms"] is not None else None
        fused_ms = max_over_ranks(rec["fused_ms"], world, dev) if rec["fused_ms"] is not None else None
        if rank == 0:
            line = {"workload": rec["workload"], "n_gpus": world, "scaling": "strong",
                    "compute_ms": compute_ms, "tflops": rec["flops"] / (compute_ms * 1e-3) / 1e12,
                    "with_gather_ms": gather_ms,
                    "tflops_with_gather": rec["flops"] / (gather_ms * 1e-3) / 1e12 if gather_ms else None,
                    "fused_gather_ms": fused_ms,
                    "tflops_fused_gather": rec["flops"] / (fused_ms * 1e-3) / 1e12 if fused_ms else None,
                    "frac_of_nominal_2250_per_gpu": rec["flops"] / (compute_ms * 1e-3) / 1e12 / world / 2250.0,
                    "kernel_config": rec["kernel_config"], "rank0_shard": rec["shard"], "iterations": args.iterations}
            text = json.dumps(line)
            print(text, flush=True)
            if args.out:
                with open(args.out, "a") as f:
                    f.write(text + "\n")
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
