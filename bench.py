#!/usr/bin/env python3
"""Benchmark of the hot paths on B200.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (all synthetic, seeded; shapes from the benchmark configurations):
  gemm8192 (default)  BF16 GEMM M=N=K=8192, operands ~ N(0,1)/sqrt(K), seed 1.  One step =
                      one launch of the GEMM on one 8192^3 problem.  With N GPUs the job is
                      C[8192, 8192*N] = A[8192,8192] . B[8192*N,8192]^T split by N-column
                      blocks: every rank owns one 8192-column slab (weak scaling, no
                      collective on the data path).
  fa_d128             FP16 attention forward B4 H32 S4096 D128, seed 2 (heads split by rank:
                      each rank owns one such problem).
  fa_d64              FP16 attention forward B16 H32 S2048 D64, seed 3.
  gemm_skinny         BF16 GEMM 128 x 4096 x 14336 (a shape of the reference's list), which the
                      default config runs as cluster split-K: HBM-bound, reported against the
                      measured copy bandwidth; five copies of B are rotated so that no step
                      finds its 117 MB in L2.

Timing: W >= 3 untimed steps, then exactly K steps between two CUDA events on the launch
stream, bracketed by barrier + synchronize; the maximum over ranks is used.  Inputs
(384 MiB for gemm8192, 512 MiB for attention) are larger than the 126 MB L2, so no flush is
needed between steps.  SM clocks and throttle reasons are sampled through NVML during the
timed region.

`value` has the inputs resident in HBM.  `e2e` is the same metric through the public
operator with HOST buffers: every step copies the inputs from pinned host memory, runs
the kernel and copies the result back, all inside the timed region; two sets of device
buffers and three streams let the upload of step i+1 and the download of step i-1 run
beside the kernel of step i.

--impl reference times the reference's CPU path for the same workload.  The reference has
no CPU implementation (its checks run cuBLAS / flash-attn on the GPU), so this is the CPU
oracle port, on all host threads, on a bounded sample of the workload per step.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "gemm8192": {"kind": "gemm", "M": 8192, "N": 8192, "K": 8192, "seed": 1,
                 "desc": "bf16 gemm M=N=K=8192, N(0,1)/sqrt(K), seed 1"},
    # HBM-bound: B (117 MB) is read once; five copies of B are rotated so that a step never
    # finds its B in the 126 MB L2.
    "gemm_skinny": {"kind": "gemm", "M": 128, "N": 4096, "K": 14336, "seed": 4, "bound": "hbm", "rotate": 5,
                    "desc": "bf16 gemm M=128 N=4096 K=14336 (split-K), N(0,1)/sqrt(K), seed 4"},
    "fa_d128": {"kind": "fa", "B": 4, "H": 32, "S": 4096, "D": 128, "seed": 2,
                "desc": "fp16 attention fwd B4 H32 S4096 D128 non-causal, N(0,1), seed 2"},
    "fa_d64": {"kind": "fa", "B": 16, "H": 32, "S": 2048, "D": 64, "seed": 3,
               "desc": "fp16 attention fwd B16 H32 S2048 D64 non-causal, N(0,1), seed 3"},
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised
# under profiles/ (null until a capture of that kernel exists).  fa_d128: the capture is the
# batch-1 slice of the workload (113.4 MB); traffic grows with the batch, so x4.
DRAM_TRAFFIC_BYTES = {"gemm8192": 1.224e9, "fa_d128": 4 * 113.4e6, "fa_d64": None, "gemm_skinny": 124.7e6}


def flops_per_step(w):
    if w["kind"] == "gemm":
        return 2.0 * w["M"] * w["N"] * w["K"]
    return 4.0 * w["B"] * w["H"] * w["S"] * w["S"] * w["D"]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p["bf16_tflops_sustained"]),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons of one GPU while a region runs."""

    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
               ("hw_thermal_slowdown", 0x40), ("hw_power_brake", 0x80), ("sync_boost", 0x10),
               ("applications_clocks", 0x2), ("display_clocks", 0x100))

    def __init__(self, index):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                for name, bit in self.REASONS:
                    if mask & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return False

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}


# ------------------------------------------------------------------ CPU path (oracle port)
def cpu_sample(wname, inputs, scale=1.0):
    """Runs the CPU oracle on a bounded sample of the workload; returns (seconds, flops,
    description).  Used as the cpu_baseline leg and as one step of --impl reference."""
    from oracle import oracle
    w = WORKLOADS[wname]
    if w["kind"] == "gemm":
        rows = min(w["M"], max(256, int(2048 * scale) // 64 * 64))
        a_bits, b_bits = inputs
        t0 = time.perf_counter()
        oracle.gemm_f64(a_bits, b_bits, row_begin=0, row_count=rows)
        dt = time.perf_counter() - t0
        return dt, 2.0 * rows * w["N"] * w["K"], f"rows 0..{rows - 1} of A against all of B ({rows}x{w['N']}x{w['K']}), fp64 accumulate"
    import numpy as np
    q, k, v = inputs
    nrows = max(32, int(256 * scale))
    rows = np.arange(0, w["S"], w["S"] // nrows, dtype=np.int32)[:nrows]
    t0 = time.perf_counter()
    oracle.attention_f32(q, k, v, False, rows=rows)
    dt = time.perf_counter() - t0
    return dt, 4.0 * w["B"] * w["H"] * nrows * w["S"] * w["D"], f"{nrows} evenly spaced query rows of every (batch, head) against all keys, fp32"


def host_inputs(wname, rank=0):
    from oracle import oracle
    w = WORKLOADS[wname]
    if w["kind"] == "gemm":
        a, _ = oracle.make_gemm_inputs(w["M"], 8, w["K"], w["seed"])                 # A: replicated
        _, b = oracle.make_gemm_inputs(8, w["N"], w["K"], w["seed"] + 1000 * rank)   # B: this rank's slab
        return a, b
    return oracle.make_fa_inputs(w["B"], w["S"], w["H"], w["D"], w["seed"] + 1000 * rank)


def run_reference(args):
    """--impl reference: the CPU port on all host threads; one step = one bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle
    oracle.use_all_cores()
    w = WORKLOADS[args.workload]
    inputs = host_inputs(args.workload)
    scale = min(1.0, 20.0 / max(args.steps, 1))   # keep the whole run within a few minutes
    for _ in range(min(args.warmup, 1)):
        cpu_sample(args.workload, inputs, scale)
    total_s, total_flops, desc = 0.0, 0.0, ""
    for _ in range(args.steps):
        dt, fl, desc = cpu_sample(args.workload, inputs, scale)
        total_s += dt
        total_flops += fl
    value = total_flops / total_s / 1e12
    cores = oracle.num_threads()
    line = {
        "impl": "reference", "metric": metric_name(w), "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_s / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64" if w["kind"] == "gemm" else "f32",
        "data": "synthetic", "config": {"workload": w["desc"], "inputs": "host memory"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU implementation of this path; this is the CPU oracle restating its semantics",
    }
    print(json.dumps(line), flush=True)
    return 0


def metric_name(w):
    return "gemm_bf16_tflops" if w["kind"] == "gemm" else "fa_fwd_fp16_tflops"


# ----------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from sm120_dl_b200 import capi, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU port)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE is {world})")
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w = WORKLOADS[args.workload]
    inputs = host_inputs(args.workload, rank)
    if w["kind"] == "gemm":
        host = [torch.from_numpy(x.view(np.int16)).view(torch.bfloat16).pin_memory() for x in inputs]
        dev_in = [t.to(dev) for t in host]
        out = torch.empty((w["M"], w["N"]), dtype=torch.bfloat16, device=dev)
        cfg = ops.gemm_config_index(args.kernel_config, w["M"], w["N"], w["K"])
        cfg_name = capi.gemm_configs()[cfg]["name"]

        # rotated copies of B for workloads smaller than L2 (kernel-only timing)
        b_copies = [dev_in[1]] + [dev_in[1].clone() for _ in range(w.get("rotate", 1) - 1)]
        turn = [0]

        def step(tensors):
            b = tensors[1]
            if tensors is dev_in:
                b = b_copies[turn[0] % len(b_copies)]
                turn[0] += 1
            ops.gemm_bf16_tn(tensors[0], b, out=out, config=cfg)
    else:
        host = [torch.from_numpy(x.view(np.int16)).view(torch.float16).pin_memory() for x in inputs]
        dev_in = [t.to(dev) for t in host]
        out = torch.empty((w["B"], w["S"], w["H"], w["D"]), dtype=torch.float16, device=dev)
        cfg = ops.fa_config_index(args.kernel_config, w["D"])
        cfg_name = capi.fa_configs()[cfg]["name"]

        def step(tensors):
            ops.flash_attn_fwd(tensors[0], tensors[1], tensors[2], out=out, config=cfg)

    flops = flops_per_step(w)
    warmup = max(args.warmup, 3)

    # ---- kernel-only: inputs resident in HBM
    for _ in range(warmup):
        step(dev_in)
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        start.record()
        for _ in range(args.steps):
            step(dev_in)
        stop.record()
        barrier()
    ms_total = start.elapsed_time(stop)
    assert capi.device_status() == 0, "a kernel reported a timed-out wait"

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region.
    # Every step copies its inputs from pinned host memory, runs the kernel and copies the
    # result back.  Two sets of device buffers and three streams let step i+1's upload and
    # step i-1's download run beside step i's kernel (PCIe is full duplex), as a caller
    # streaming problems through the operator would do; nothing is skipped or reused.
    e2e_steps = max(2, min(args.steps, 10))
    depth = 2
    host_out = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(depth)]
    stage = [[torch.empty_like(t) for t in dev_in] for _ in range(depth)]
    outs = [torch.empty_like(out) for _ in range(depth)]
    s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    uploaded = [torch.cuda.Event() for _ in range(depth)]
    computed = [torch.cuda.Event() for _ in range(depth)]
    downloaded = [torch.cuda.Event() for _ in range(depth)]

    def run_into(tensors, dst):
        if w["kind"] == "gemm":
            ops.gemm_bf16_tn(tensors[0], tensors[1], out=dst, config=cfg)
        else:
            ops.flash_attn_fwd(tensors[0], tensors[1], tensors[2], out=dst, config=cfg)

    def e2e_step(i):
        b = i % depth
        with torch.cuda.stream(s_in):
            s_in.wait_event(computed[b])        # the kernel of step i-2 has read these buffers
            for d, h in zip(stage[b], host):
                d.copy_(h, non_blocking=True)
            uploaded[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(uploaded[b])
            s_run.wait_event(downloaded[b])     # the download of step i-2 has read this output
            run_into(stage[b], outs[b])
            computed[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(computed[b])
            host_out[b].copy_(outs[b], non_blocking=True)
            downloaded[b].record(s_out)

    def e2e_run(n):
        for s in (s_in, s_run, s_out):
            s.wait_stream(torch.cuda.current_stream(dev))
        for i in range(n):
            e2e_step(i)
        for s in (s_in, s_run, s_out):
            torch.cuda.current_stream(dev).wait_stream(s)

    e2e_run(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    assert capi.device_status() == 0, "a kernel reported a timed-out wait"

    times = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = (float(x) for x in times.cpu())

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms_total / args.steps
        per_gpu_tflops = flops / (ms_per_step * 1e-3) / 1e12
        value = per_gpu_tflops * world
        e2e_value = flops * world / (e2e_ms / e2e_steps * 1e-3) / 1e12
        # A region of a few tens of milliseconds sits between the burst and the sustained
        # library figure; the burst one is the stricter denominator.
        peak = peaks["bf16_tflops"]
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = host_out[0].numel() * host_out[0].element_size()
        if w.get("bound") == "hbm":
            nbytes = 2.0 * (w["M"] * w["K"] + w["N"] * w["K"] + w["M"] * w["N"])
            gbs = nbytes / (ms_per_step * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} hbm_gbs (copy)",
                        "frac_of_nominal_8000": gbs / 8000.0, "traffic": DRAM_TRAFFIC_BYTES.get(args.workload)}
            l2_note = "B rotated over %d copies (%d MB) so no step finds it in L2" % (
                w["rotate"], w["rotate"] * w["N"] * w["K"] * 2 // 2 ** 20)
        else:
            roofline = {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peak, "unit": "TFLOP/s",
                        "frac": per_gpu_tflops / peak, "peak_source": f"{peaks['source']} bf16_tflops (burst)",
                        "frac_of_nominal_2250": per_gpu_tflops / 2250.0,
                        "traffic": DRAM_TRAFFIC_BYTES.get(args.workload)}
            l2_note = "inputs larger than L2, no flush between steps"
        line = {
            "metric": metric_name(w), "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if w["kind"] == "gemm" else "fp16", "data": "synthetic",
            "config": {"workload": w["desc"], "kernel_config": cfg_name,
                       "parallelism": "1 gpu" if world == 1 else f"{world} ranks, one problem slab per rank, no collective",
                       "l2": l2_note},
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "gpu_launches": e2e_steps, "pipeline": "2 buffer sets; upload, kernel and download on 3 streams"},
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
        }
        if not args.no_cpu_baseline:
            from oracle import oracle
            oracle.use_all_cores()
            dt, fl, desc = cpu_sample(args.workload, inputs)
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.num_threads(),
                                    "kind": "port", "sample": desc, "seconds": dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="gemm8192")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--kernel-config", default=None, help="config name instead of the library's default for the shape")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (N=1 only has it anyway)")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("--steps must be >= 1")
    if args.impl == "reference":
        return run_reference(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        args.no_cpu_baseline = True   # the CPU leg runs at N=1 only
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
