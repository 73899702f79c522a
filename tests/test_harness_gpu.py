"""GPU tests of the test_gemm_cute harness: the reference's command lines must work and
print the reference's line formats (gemm/test.cpp:1242-1303, :765-786 of HugeOrca/sm120-dl)."""

import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "sm120_dl_b200", "gemm", "test_gemm_cute")


@pytest.fixture(scope="module")
def exe(cuda_device):
    from sm120_dl_b200 import build
    build.build_lib()
    build.build_test_gemm_cute()
    return EXE


def _run(exe, *args, timeout=600):
    return subprocess.run([exe, *args], capture_output=True, text=True, timeout=timeout)


def test_shape_mode_verifies_against_cublas_then_ranks(exe):
    p = _run(exe, "1024", "1024", "1024")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert re.search(r"\{1024, 1024, 1024\} verify summary: passed=\d+ failed=0 skipped=\d+ total=\d+", p.stdout)
    assert "{1024, 1024, 1024} verify success: bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8" in p.stdout
    assert re.search(r"^BEST: 1024,1024,1024 bf16_\S+   \d+\.\d{4} ms \d+\.\d{3} TFLOP/s cublas \d+\.\d{4} ms "
                     r"\d+\.\d{3} TFLOP/s gemm_tn/cublas=\d+\.\d{2}%$", p.stdout, re.M)
    assert re.search(r"^   1\. bf16_", p.stdout, re.M)


def test_skipped_configs_are_reported(exe):
    p = _run(exe, "128", "4096", "512")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "{128, 4096, 512} verify skipped: bf16_bm256_" in p.stdout
    assert re.search(r"verify summary: passed=\d+ failed=0 skipped=[1-9]\d* ", p.stdout)


def test_func_mode_with_prefix_and_pattern(exe):
    p = _run(exe, "--func", "gemm_tn_bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "--verify")
    assert p.returncode == 0, p.stdout + p.stderr
    assert "func config=bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8 mode=verify M=4096 N=4096 K=4096 warmup=5 iterations=25" in p.stdout
    assert re.search(r"verify detail: max_abs=\S+ max_rel=\S+ max_idx=\d+ mismatches=0/16777216", p.stdout)
    p = _run(exe, "--func", "bf16_bm128_bn128_bk64_s5*", "--benchmark")
    assert p.returncode == 0 and "TFLOP/s cublas" in p.stdout
    p = _run(exe, "--func", "bf16_bm256_bn256*")
    assert p.returncode != 0 and "ambiguous config pattern" in p.stderr
    p = _run(exe, "--func", "no_such")
    assert p.returncode != 0 and "unknown config: no_such" in p.stderr and "available configs:" in p.stderr


def test_profile_and_usage(exe):
    p = _run(exe, "--profile", "bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "2048", "2048", "2048", "2")
    assert p.returncode == 0 and "profile config=bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8 M=2048 N=2048 K=2048 warmup=2" in p.stdout
    p = _run(exe, "--profile", "bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "100", "2048", "2048")
    assert p.returncode != 0 and "profile skipped:" in p.stdout
    p = _run(exe)
    assert p.returncode != 0 and p.stderr.startswith("usage:")
    p = _run(exe, "12", "x", "5")
    assert p.returncode != 0 and "usage:" in p.stderr


def test_verify_host_mode(exe):
    p = _run(exe, "--verify-host", "512", "512", "512")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "verify-host success" in p.stdout and "failed" not in p.stdout


def test_registry_run_still_refuses_shapes_its_tile_does_not_divide(exe):
    """The C ABI accepts ragged shapes, the reference-shaped registry keeps gemm_tn's rule."""
    p = _run(exe, "--profile", "bf16_bm128_bn64_bk64_s8_cta1_acc2_bsw8", "130", "64", "64")
    assert p.returncode != 0 and "profile skipped:" in p.stdout
