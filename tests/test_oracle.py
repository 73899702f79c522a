"""CPU tests of the oracle itself: the C++ code against the committed fixtures (made by
independent torch-CPU float64 implementations, tests/golden/make_golden.py) and against
the numpy restatement, plus the comparison rule and the seeded generators."""

import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _fixtures(prefix):
    files = sorted(glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))
    assert files, "fixtures missing: run python tests/golden/make_golden.py"
    return files


@pytest.mark.parametrize("path", _fixtures("gemm_"), ids=os.path.basename)
def test_gemm_oracle_matches_golden(oracle, path):
    fx = np.load(path)
    M, N, K = (int(x) for x in fx["shape"])
    a, b = oracle.make_gemm_inputs(M, N, K, int(fx["seed"]), str(fx["dist"]))
    got = oracle.gemm_f64(a, b)
    # products of bf16 values are exact in double; only the summation order may differ
    np.testing.assert_allclose(got, fx["expected"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(oracle.gemm_numpy(a, b), fx["expected"], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("path", _fixtures("attention_"), ids=os.path.basename)
def test_attention_oracle_matches_golden(oracle, path):
    fx = np.load(path)
    B, S, H, D = (int(x) for x in fx["shape"])
    q, k, v = oracle.make_fa_inputs(B, S, H, D, int(fx["seed"]))
    causal = bool(fx["causal"])
    got = oracle.attention_f32(q, k, v, causal)
    assert got.shape == (B, S, H, D)
    # the oracle works in fp32; the fixture was computed in float64
    assert np.abs(got - fx["expected"]).max() < 5e-6
    assert np.abs(oracle.attention_numpy(q, k, v, causal) - fx["expected"]).max() < 5e-6


def test_gemm_row_subset_equals_full(oracle):
    a, b = oracle.make_gemm_inputs(70, 52, 136, 4)
    full = oracle.gemm_f64(a, b)
    part = oracle.gemm_f64(a, b, row_begin=13, row_count=40)
    np.testing.assert_array_equal(part, full[13:53])


def test_attention_row_subset_and_strides(oracle):
    q, k, v = oracle.make_fa_inputs(2, 77, 4, 64, 9)
    full = oracle.attention_f32(q, k, v, causal=True)
    rows = np.array([0, 1, 40, 76], dtype=np.int32)
    np.testing.assert_allclose(oracle.attention_f32(q, k, v, causal=True, rows=rows), full[:, rows], atol=1e-7)
    # a head slice is a strided view; the oracle must address it through the strides
    sl = oracle.attention_f32(q[:, :, 1:3], k[:, :, 1:3], v[:, :, 1:3], causal=True)
    np.testing.assert_allclose(sl, full[:, :, 1:3], atol=1e-7)


def test_causal_first_row_is_v0(oracle):
    q, k, v = oracle.make_fa_inputs(1, 16, 2, 64, 1)
    out = oracle.attention_f32(q, k, v, causal=True)
    np.testing.assert_allclose(out[:, 0], v.view(np.float16)[:, 0].astype(np.float32), atol=1e-6)


def test_compare_rule(oracle):
    ref = np.array([0.0, 1.0, -2.0, 100.0])
    ok = oracle.compare(ref + np.array([0.009, 0.05, -0.1, 4.9]), ref, 1e-2, 5e-2)
    assert ok["passed"] and ok["mismatches"] == 0
    bad = oracle.compare(ref + np.array([0.011, 0.0, 0.0, 0.0]), ref, 1e-2, 5e-2)
    assert not bad["passed"] and bad["first_bad"] == 0 and bad["mismatches"] == 1
    nan = oracle.compare(np.array([np.nan, 1.0, -2.0, 100.0]), ref, 1e-2, 5e-2)
    assert not nan["passed"]
    # bounded relative error divides by max(|ref|, rms(ref)), not by a near-zero reference
    st = oracle.compare(ref + 0.5, ref, 10.0, 0.0)
    rms = np.sqrt((ref ** 2).mean())
    assert abs(st["max_rel_bounded"] - 0.5 / rms) < 1e-12


def test_generators_are_deterministic_and_rounded(oracle):
    a1, b1 = oracle.make_gemm_inputs(8, 8, 64, 0, "uniform1")
    a2, b2 = oracle.make_gemm_inputs(8, 8, 64, 0, "uniform1")
    np.testing.assert_array_equal(a1, a2)
    np.testing.assert_array_equal(b1, b2)
    vals = oracle.f32_from_bf16_bits(a1)
    assert np.abs(vals).max() <= 1.0 and (vals.view(np.uint32) & 0xFFFF == 0).all()
    # bf16 rounding is round-to-nearest-even
    x = np.array([1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8, -(1.0 + 2 ** -8)], dtype=np.float32)
    np.testing.assert_array_equal(oracle.f32_from_bf16_bits(oracle.bf16_bits_from_f32(x)),
                                  np.array([1.0, 1.0 + 2 ** -6, -1.0], dtype=np.float32))
    q1 = oracle.make_fa_inputs(1, 4, 1, 64, 2)[0]
    q2 = oracle.make_fa_inputs(1, 4, 1, 64, 2)[0]
    np.testing.assert_array_equal(q1, q2)
