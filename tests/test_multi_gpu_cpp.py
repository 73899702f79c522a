"""The C++ multi-GPU driver (sm120_dl_b200/gemm/test_gemm_multi_gpu): N-column shards on every
GPU of the box, compute-only, epilogue-fused gather through peer-mapped pointers and the NCCL
gather, with the gathered C checked against cuBLAS inside the program.  Needs two GPUs; on a
one-GPU box only the argument handling and the single-device path run."""

import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "sm120_dl_b200", "gemm", "test_gemm_multi_gpu")


def _run(args):
    return subprocess.run([BINARY] + args, capture_output=True, text=True, timeout=600)


def test_cpp_driver_shards_and_gathers(cuda_device):
    import torch
    assert os.path.exists(BINARY), "build it with `python -m sm120_dl_b200.build test_gemm_multi_gpu`"
    gpus = min(torch.cuda.device_count(), 8)
    # N must split into 256-column blocks per GPU
    p = _run(["--gpus", str(gpus), "--iterations", "3", "4096", str(256 * gpus * 2), "2048"])
    assert p.returncode == 0, p.stdout + p.stderr
    line = [x for x in p.stdout.splitlines() if x.startswith("multi_gpu ")][-1]
    assert "verify=PASS" in line and f"gpus={gpus}" in line, line
    for key in ("compute_ms", "fused_gather_ms", "nccl_gather_ms"):
        assert float(re.search(key + r"=([0-9.]+)", line).group(1)) > 0.0
    # bad arguments end with a usage message, not a launch
    p = _run(["--gpus", "99"])
    assert p.returncode == 1 and "GPUs" in p.stderr
    p = _run(["--gpus", str(gpus), "1024", "1000", "512"])
    assert p.returncode == 1 and "multiple of 256" in p.stderr
