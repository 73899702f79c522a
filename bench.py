#!/usr/bin/env python3
"""Benchmark of the two hot paths on B200.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

The headline (`metric`, `value`, `ms_per_step`, `roofline`, `e2e`, `cpu_baseline`) is the
workload named by --workload, by default the BF16 GEMM 8192^3:

  gemm8192 (default)  BF16 GEMM M=N=K=8192, operands ~ N(0,1)/sqrt(K), seed 1.  One step =
                      one launch of the GEMM on one 8192^3 problem.  With N GPUs the job is
                      C[8192, 8192*N] = A[8192,8192] . B[8192*N,8192]^T split by N-column
                      blocks: every rank owns one 8192-column slab (weak scaling, no
                      collective on the data path).
  fa_d128             FP16 attention forward B4 H32 S4096 D128, seed 2 (one such problem per
                      rank).
  fa_d64              FP16 attention forward B16 H32 S2048 D64, seed 3.
  gemm_skinny         BF16 GEMM 128 x 4096 x 14336 (a shape of the reference's list), which the
                      default config runs as cluster split-K: HBM-bound, reported against the
                      measured copy bandwidth; five copies of B are rotated so that no step
                      finds its 117 MB in L2.

The same line carries, measured in the same run (unless --no-extras):

  sustained   the headline kernel launched back to back for >= 2 s, with the median SM clock
              and power sampled over that region, beside the library's sustained figure
  fa_d128, fa_d64
              the two attention configurations (value, ms_per_step, roofline, clocks)
  config5     the fixed-size problems of the multi-GPU configuration split over the N ranks
              (strong scaling): BF16 GEMMs M=16384 with (N,K) in {(4096,4096), (14336,4096),
              (4096,14336)} by N-column blocks and FP16 attention B1 H64 S32768 D128 by
              heads; per problem the compute-only rate, and for N > 1 the rate with the
              NCCL all-gather and with the gather fused into the kernel's epilogue.  Times
              are CUDA-event times, maximum over ranks.

Timing: W >= 3 untimed steps, then exactly K steps between two CUDA events on the launch
stream, bracketed by barrier + synchronize; the maximum over ranks is used.  Inputs
(384 MiB for gemm8192, 512 MiB for attention) are larger than the 126 MB L2, so no flush is
needed between steps.  SM clocks and throttle reasons are sampled through NVML during every
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
import glob
import json
import os
import re
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

CONFIG5_GEMMS = [(16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336)]
CONFIG5_ATTENTION = (1, 32768, 64, 128)   # B, S, H, D
SUSTAINED_SECONDS = 2.0
NOMINAL_TFLOPS = 2250.0
EX2_PER_CLOCK_PER_SM = 16


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


def profiled_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of each workload's kernel, as
    recorded in the ncu summaries under profiles/ (a line `workload=<name>
    dram_bytes_per_launch=<bytes>` written beside the command that produced the capture).
    A workload without a capture has no entry."""
    found = {}
    pat = re.compile(r"workload=(\w+)\s+dram_bytes_per_launch=([0-9.eE+]+)")
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        try:
            with open(path, errors="replace") as f:
                for m in pat.finditer(f.read()):
                    found[m.group(1)] = {"bytes": float(m.group(2)), "source": os.path.relpath(path, ROOT)}
        except OSError:
            pass
    return found


class ClockSampler:
    """Polls NVML for SM clock, power and throttle reasons of one GPU while a region runs."""

    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
               ("hw_thermal_slowdown", 0x40), ("hw_power_brake", 0x80), ("sync_boost", 0x10),
               ("applications_clocks", 0x2), ("display_clocks", 0x100))

    def __init__(self, index, period=0.002):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self.period = period
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
            time.sleep(self.period)

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
                "power_w_max": max(self.power) if self.power else None,
                "power_w_median": statistics.median(self.power) if self.power else None}


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
    from sm120_dl_b200 import synthetic
    w = WORKLOADS[wname]
    if w["kind"] == "gemm":
        a, _ = synthetic.make_gemm_inputs(w["M"], 8, w["K"], w["seed"])                 # A: replicated
        _, b = synthetic.make_gemm_inputs(8, w["N"], w["K"], w["seed"] + 1000 * rank)   # B: this rank's slab
        return a, b
    return synthetic.make_fa_inputs(w["B"], w["S"], w["H"], w["D"], w["seed"] + 1000 * rank)


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
class Bench:
    """State shared by the legs of the GPU arm: device, ranks, launch counter."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU port)")
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            if self.world == 1 and args.gpus > 1:
                raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE is {self.world})")
            args.gpus = self.world
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.launches = 0
        self.peaks = measured_peaks()
        self.traffic = profiled_traffic()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, *values):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.cpu()]

    def timed(self, fn, steps, warmup):
        """(total ms of `steps` calls, clock summary): CUDA events on the launch stream
        between barrier + synchronize, clocks sampled over the region."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(self.local_rank) as clocks:
            start.record()
            for _ in range(steps):
                fn()
            stop.record()
            self.barrier()
        self.launches += steps
        return start.elapsed_time(stop), clocks.summary()


def make_workload(bench, wname, kernel_config):
    """Device tensors and the step function of one workload."""
    import numpy as np
    from sm120_dl_b200 import capi, ops
    torch, dev = bench.torch, bench.dev
    w = WORKLOADS[wname]
    inputs = host_inputs(wname, bench.rank)
    if w["kind"] == "gemm":
        host = [torch.from_numpy(x.view(np.int16)).view(torch.bfloat16).pin_memory() for x in inputs]
        dev_in = [t.to(dev) for t in host]
        out = torch.empty((w["M"], w["N"]), dtype=torch.bfloat16, device=dev)
        cfg = ops.gemm_config_index(kernel_config, w["M"], w["N"], w["K"])
        cfg_name = capi.gemm_configs()[cfg]["name"]
        # rotated copies of B for workloads smaller than L2 (kernel-only timing)
        b_copies = [dev_in[1]] + [dev_in[1].clone() for _ in range(w.get("rotate", 1) - 1)]
        turn = [0]

        def step():
            b = b_copies[turn[0] % len(b_copies)]
            turn[0] += 1
            ops.gemm_bf16_tn(dev_in[0], b, out=out, config=cfg)

        def run_into(tensors, dst):
            ops.gemm_bf16_tn(tensors[0], tensors[1], out=dst, config=cfg)
    else:
        host = [torch.from_numpy(x.view(np.int16)).view(torch.float16).pin_memory() for x in inputs]
        dev_in = [t.to(dev) for t in host]
        out = torch.empty((w["B"], w["S"], w["H"], w["D"]), dtype=torch.float16, device=dev)
        cfg = ops.fa_config_index(kernel_config, w["D"])
        cfg_name = capi.fa_configs()[cfg]["name"]

        def step():
            ops.flash_attn_fwd(dev_in[0], dev_in[1], dev_in[2], out=out, config=cfg)

        def run_into(tensors, dst):
            ops.flash_attn_fwd(tensors[0], tensors[1], tensors[2], out=dst, config=cfg)
    return {"w": w, "inputs": inputs, "host": host, "dev_in": dev_in, "out": out, "cfg_name": cfg_name,
            "step": step, "run_into": run_into}


def roofline_of(bench, wname, w, per_gpu_rate, ms_per_step, clocks):
    peaks = bench.peaks
    traffic = bench.traffic.get(wname)
    if w.get("bound") == "hbm":
        nbytes = 2.0 * (w["M"] * w["K"] + w["N"] * w["K"] + w["M"] * w["N"])
        gbs = nbytes / (ms_per_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} hbm_gbs (copy)",
                "frac_of_nominal_8000": gbs / 8000.0, "traffic": traffic["bytes"] if traffic else None,
                "traffic_source": traffic["source"] if traffic else None}
    # A region of tens of milliseconds sits between the burst and the sustained library
    # figure; the burst one is the stricter denominator.
    r = {"bound": "tensor", "achieved": per_gpu_rate, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
         "frac": per_gpu_rate / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} bf16_tflops (burst)",
         "frac_of_nominal_2250": per_gpu_rate / NOMINAL_TFLOPS,
         "traffic": traffic["bytes"] if traffic else None, "traffic_source": traffic["source"] if traffic else None}
    if w["kind"] == "fa":
        # the other unit this kernel leans on: one ex2 per score, 16 per clock per SM
        ex2 = float(w["B"]) * w["H"] * w["S"] * w["S"]
        sms = bench.torch.cuda.get_device_properties(bench.dev).multi_processor_count
        mhz = clocks.get("sm_max_mhz") or 1965
        peak = EX2_PER_CLOCK_PER_SM * sms * mhz * 1e6
        r["sfu"] = {"ex2_per_s": ex2 / (ms_per_step * 1e-3), "peak_ex2_per_s_at_max_clock": peak,
                    "frac": ex2 / (ms_per_step * 1e-3) / peak,
                    "note": "exponentials evaluated by the FMA-pipe polynomial count as ex2 here"}
    return r


def measure_workload(bench, wname, args, kernel_config=None):
    """Kernel-only timing of one workload: a sub-record of the JSON line."""
    wl = make_workload(bench, wname, kernel_config)
    w = wl["w"]
    warmup = max(args.warmup, 3)
    ms_total, clocks = bench.timed(wl["step"], args.steps, warmup)
    (ms_total,) = bench.max_over_ranks(ms_total)
    ms_per_step = ms_total / args.steps
    per_gpu = flops_per_step(w) / (ms_per_step * 1e-3) / 1e12
    rec = {"metric": metric_name(w), "value": per_gpu * bench.world, "unit": "TFLOP/s", "ms_per_step": ms_per_step,
           "steps": args.steps, "warmup": warmup, "workload": w["desc"], "kernel_config": wl["cfg_name"],
           "roofline": roofline_of(bench, wname, w, per_gpu, ms_per_step, clocks), "clocks": clocks}
    return wl, rec


def sustained_leg(bench, wl, ms_per_step):
    """The headline kernel back to back for >= SUSTAINED_SECONDS, clocks sampled."""
    n = max(10, int(SUSTAINED_SECONDS * 1e3 / ms_per_step) + 1)
    ms_total, clocks = bench.timed(wl["step"], n, 0)
    (ms_total,) = bench.max_over_ranks(ms_total)
    rate = flops_per_step(wl["w"]) * n / (ms_total * 1e-3) / 1e12
    rec = {"seconds": ms_total * 1e-3, "launches": n, "value": rate * bench.world, "per_gpu": rate, "unit": "TFLOP/s",
           "ms_per_step": ms_total / n, "clocks": clocks,
           "library_sustained_tflops": bench.peaks["bf16_tflops_sustained"],
           "frac_of_library_sustained": rate / bench.peaks["bf16_tflops_sustained"],
           "frac_of_nominal_2250": rate / NOMINAL_TFLOPS}
    mhz = clocks.get("sm_mhz")
    if mhz:
        # time x median clock: what the same launch would take in cycles, independent of the
        # clock the power cap allowed
        rec["mcycles_per_step"] = ms_total / n * 1e-3 * mhz
        rec["tflops_at_max_clock"] = rate * (clocks.get("sm_max_mhz") or mhz) / mhz
    return rec


def e2e_leg(bench, wl, args):
    """Host buffers in, host buffer out, copies inside the timed region.  Every step copies
    its inputs from pinned host memory, runs the kernel and copies the result back.  Two sets
    of device buffers and three streams let step i+1's upload and step i-1's download run
    beside step i's kernel (PCIe is full duplex), as a caller streaming problems through the
    operator would do; nothing is skipped or reused."""
    torch, dev = bench.torch, bench.dev
    host, dev_in, out = wl["host"], wl["dev_in"], wl["out"]
    e2e_steps = max(2, min(args.steps, 10))
    depth = 2
    host_out = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(depth)]
    stage = [[torch.empty_like(t) for t in dev_in] for _ in range(depth)]
    outs = [torch.empty_like(out) for _ in range(depth)]
    s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    uploaded = [torch.cuda.Event() for _ in range(depth)]
    computed = [torch.cuda.Event() for _ in range(depth)]
    downloaded = [torch.cuda.Event() for _ in range(depth)]

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
            wl["run_into"](stage[b], outs[b])
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
    bench.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    bench.barrier()
    (e2e_ms,) = bench.max_over_ranks(e0.elapsed_time(e1))
    bench.launches += e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = host_out[0].numel() * host_out[0].element_size()
    value = flops_per_step(wl["w"]) * bench.world / (e2e_ms / e2e_steps * 1e-3) / 1e12
    return {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": e2e_steps, "gpu_launches": e2e_steps,
            "pipeline": "2 buffer sets; upload, kernel and download on 3 streams"}


def config5_leg(bench, args):
    """The multi-GPU configuration's fixed-size problems split over the ranks of this job."""
    from sm120_dl_b200 import capi, sweep
    iterations = max(3, min(args.steps, 10))
    records = []
    jobs = [("gemm", shape) for shape in CONFIG5_GEMMS] + [("attention", None)]
    for kind, shape in jobs:
        if kind == "gemm":
            rec = sweep.run_gemm(*shape, bench.world, bench.rank, bench.dev, iterations)
        else:
            rec = sweep.run_attention(bench.world, bench.rank, bench.dev, iterations)
        panel = rec.get("panel_gather_ms")
        n_variants = 1 + (rec["gather_ms"] is not None) + (rec["fused_ms"] is not None) + 4 * (panel is not None)
        bench.launches += n_variants * iterations
        compute_ms, gather_ms, fused_ms, panel_ms = bench.max_over_ranks(
            rec["compute_ms"], rec["gather_ms"] or 0.0, rec["fused_ms"] or 0.0, panel or 0.0)
        rate = lambda ms: rec["flops"] / (ms * 1e-3) / 1e12 if ms > 0 else None  # noqa: E731
        records.append({
            "workload": rec["workload"], "scaling": "strong", "n_gpus": bench.world, "iterations": iterations,
            "kernel_config": rec["kernel_config"], "rank0_shard": rec["shard"],
            "compute_ms": compute_ms, "tflops": rate(compute_ms),
            "frac_of_nominal_2250_per_gpu": rate(compute_ms) / bench.world / NOMINAL_TFLOPS,
            "nccl_gather_ms": gather_ms or None, "tflops_nccl_gather": rate(gather_ms),
            "nccl_gather_4_row_panels_ms": panel_ms or None,
            "fused_gather_ms": fused_ms or None, "tflops_fused_gather": rate(fused_ms)})
        bench.torch.cuda.empty_cache()
    assert capi.device_status() == 0, "a kernel reported a timed-out wait"
    return records


def run_gpu(args):
    from sm120_dl_b200 import capi
    bench = Bench(args)
    wl, head = measure_workload(bench, args.workload, args, args.kernel_config)
    assert capi.device_status() == 0, "a kernel reported a timed-out wait"
    w = wl["w"]
    extras = {}
    if not args.no_extras:
        extras["sustained"] = sustained_leg(bench, wl, head["ms_per_step"])
    e2e = e2e_leg(bench, wl, args)
    assert capi.device_status() == 0, "a kernel reported a timed-out wait"
    inputs = wl["inputs"]
    del wl
    bench.torch.cuda.empty_cache()
    if not args.no_extras:
        for other in ("fa_d128", "fa_d64", "gemm8192"):
            if other == args.workload:
                continue
            wl2, rec = measure_workload(bench, other, args)
            if other == "fa_d128":
                # attention runs into the same power cap as the GEMM: say at which clock
                rec["sustained"] = sustained_leg(bench, wl2, rec["ms_per_step"])
            del wl2
            bench.torch.cuda.empty_cache()
            extras[other] = rec
        assert capi.device_status() == 0, "a kernel reported a timed-out wait"
        extras["config5"] = config5_leg(bench, args)

    if bench.rank == 0:
        world = bench.world
        l2_note = ("B rotated over %d copies so no step finds it in L2" % w["rotate"] if w.get("rotate")
                   else "inputs larger than L2, no flush between steps")
        line = {
            "metric": head["metric"], "value": head["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": head["warmup"], "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if w["kind"] == "gemm" else "fp16", "data": "synthetic",
            "config": {"workload": w["desc"], "kernel_config": head["kernel_config"],
                       "parallelism": "1 gpu" if world == 1 else f"{world} ranks, one problem slab per rank, no collective",
                       "l2": l2_note},
            "roofline": head["roofline"],
            "e2e": e2e,
            "gpu_launches": bench.launches,
            "clocks": head["clocks"],
        }
        line.update(extras)
        if not args.no_cpu_baseline:
            from oracle import oracle
            oracle.use_all_cores()
            dt, fl, desc = cpu_sample(args.workload, inputs)
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.num_threads(),
                                    "kind": "port", "sample": desc, "seconds": dt}
        print(json.dumps(line), flush=True)
    if bench.world > 1:
        bench.dist.barrier()
        bench.dist.destroy_process_group()
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
    ap.add_argument("--no-extras", action="store_true",
                    help="headline workload only: no sustained leg, attention sub-records or config5")
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
