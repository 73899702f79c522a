"""GPU smoke tests of the drop-in scripts (same command lines as the reference's)."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FA = os.path.join(ROOT, "sm120_dl_b200", "flashattention")


@pytest.fixture(scope="module")
def built(cuda_device):
    from sm120_dl_b200 import build
    build.build_all()


def _py(script, *args, cwd=FA, timeout=600):
    return subprocess.run([sys.executable, script, *args], cwd=cwd, capture_output=True, text=True, timeout=timeout)


def test_verify_case_and_default_list_prefix(built):
    p = _py("verify.py", "--case", "256", "128", "4", "1", "1", "--tight")
    assert p.returncode == 0, p.stdout + p.stderr
    assert p.stdout.startswith("PASS b1_hn4_seq256_hd128_casual1 max_abs=")
    p = _py("verify.py", "--case", "100", "64", "1", "1", "0")
    assert p.returncode == 1 and "seq_len must be a multiple of 64" in p.stdout


def test_verify_all_configs(built):
    p = _py("verify.py", "--all")
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-2000:]
    assert "SUMMARY kernel_templates passed=" in p.stdout and "FAIL" not in p.stdout


def test_benchmark_case_writes_summary(built):
    p = _py("benchmark.py", "--case", "2048", "64", "16", "1", "--iterations", "5", "--warmup", "2")
    assert p.returncode == 0, p.stdout + p.stderr
    assert "custom/official:" in p.stdout and "b1_hn16_seq2048_hd64_casual0" in p.stdout
    assert os.path.exists(os.path.join(FA, "benchmark.txt"))


def test_compute_rate_script_lists_and_runs(built):
    p = _py("test_compute_rate.py", "--list-names")
    assert p.returncode == 0 and "hd128_" in p.stdout and "hd64_" in p.stdout
    name = [n for n in p.stdout.split() if n.startswith("hd64_")][0]
    p = _py("test_compute_rate.py", "--func", name, "--seq-len", "512", "--head-num", "4", "--batch", "1", "--sleep", "0")
    assert p.returncode == 0 and "PROFILE func=" in p.stdout and "DONE func=" in p.stdout


def test_single_case_runner(built):
    p = _py("test.py")
    assert p.returncode == 0 and " hd=128 bm=64 bn=64 " in p.stdout
    name = [line.split()[0] for line in p.stdout.splitlines() if line.startswith("hd128_")][0]
    p = _py("test.py", "--config", "b2_hn4_seq512_hd128_casual1", "--func", name)
    assert p.returncode == 0, p.stdout + p.stderr
    assert p.stdout.startswith(f"RUN b2_hn4_seq512_hd128_casual1 func={name}")
    assert "DONE b2_hn4_seq512_hd128_casual1" in p.stdout and "output_shape=(2, 512, 4, 128)" in p.stdout
    p = _py("test.py", "--config", "512", "64", "4", "2", "0", "--func", name)
    assert p.returncode != 0 and "expects head_dim=128, got 64" in p.stderr
