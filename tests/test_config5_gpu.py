"""GPU parity tests of the multi-GPU configuration's problems and of the large entries of the
reference's attention shape list, on ONE GPU: what a rank of an 8-GPU job computes is a column
slab (GEMM) or a head slice (attention) of the full problem, addressed through leading
dimensions / strides, and that is what runs here, through the C ABI, against the CPU oracle.

  BF16 GEMM M=16384, (N,K) in {(4096,4096), (14336,4096), (4096,14336)}, N(0,1)/sqrt(K),
  seed 4: the whole problem (three seeded 64-row bands and the column-sum property) and the
  slab of width N/8 that rank 3 of 8 writes into a full-width C.
  FP16 attention B=1 H=64 S=32768 D=128, N(0,1), seed 5: one 8-head slice of full tensors.
  Attention shapes (seq, head_dim, heads, batch) of flashattention/v3_mMnNkN/verify.py:26-45
  with S >= 2048, causal off and on, every softmax layout.

Tolerances are the suite's: GEMM |d| <= 1e-2 + 5e-2 |ref| and bounded relative error
<= 1e-2; attention max |d| <= 2e-3."""

import ctypes
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ABS_BOUND = 2e-3


@pytest.fixture(scope="module")
def env(cuda_device, oracle):
    import torch
    from sm120_dl_b200 import capi
    return torch, capi, capi.lib(), oracle, cuda_device


def _layout_defaults(capi, head_dim):
    """Index of the first config of every softmax layout for this head_dim."""
    first = {}
    for i, cfg in enumerate(capi.fa_configs()):
        if cfg["head_dim"] == head_dim:
            first.setdefault(cfg["softmax_layout"], i)
    return sorted(first.values())


def _gemm(env, cfg, a, b, c, M, N, K, ldc):
    torch, capi, lib, _, _ = env
    rc = lib.b200_gemm_bf16_tn(cfg, M, N, K, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), c.data_ptr(), ldc, None)
    assert rc == 0, lib.b200_last_error().decode()
    assert capi.device_status() == 0


def _check_gemm(oracle, got, ref):
    st = oracle.compare(got, ref, 1e-2, 5e-2)
    assert st["passed"] and st["max_rel_bounded"] <= 1e-2, st


@pytest.mark.parametrize("shape", [(16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336)],
                         ids=lambda s: "%dx%dx%d" % s)
def test_config5_gemm_full_and_column_slab(env, shape):
    torch, capi, lib, oracle, dev = env
    M, N, K = shape
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 4)
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    _gemm(env, lib.b200_gemm_default_config(M, N, K), a, b, c, M, N, K, N)
    rng = np.random.Generator(np.random.PCG64(4))
    bands = [int(r) * 64 for r in sorted(rng.choice(M // 64, size=3, replace=False))]
    refs = {r0: oracle.gemm_f64(a_bits, b_bits, row_begin=r0, row_count=64) for r0 in bands}
    for r0 in bands:
        _check_gemm(oracle, c[r0:r0 + 64].float().cpu().numpy(), refs[r0])
    # size-independent: column sums of C equal (sum of A's rows) @ B^T
    col_sums = c.double().sum(dim=0).cpu().numpy()
    a_sum = oracle.f32_from_bf16_bits(a_bits).astype(np.float64).sum(axis=0)
    expect = oracle.f32_from_bf16_bits(b_bits).astype(np.float64) @ a_sum
    assert np.abs(col_sums - expect).max() <= 2e-3 * np.sqrt(M) * c.float().abs().max().item()

    # what rank 3 of 8 does: columns [3N/8, 4N/8) written into a full-width C (ldc = N) with
    # the config the library picks for the slab's shape; the rest of C stays untouched
    width = N // 8
    n0 = 3 * width
    full = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    _gemm(env, lib.b200_gemm_default_config(M, width, K), a, b[n0:n0 + width], full[:, n0:], M, width, K, N)
    for r0 in bands:
        _check_gemm(oracle, full[r0:r0 + 64, n0:n0 + width].float().cpu().numpy(), refs[r0][:, n0:n0 + width])
    outside = torch.cat([full[:, :n0], full[:, n0 + width:]], dim=1)
    assert bool(torch.isnan(outside.float()).all()), "the slab call wrote outside its columns"


def _fa(env, cfg, q, k, v, causal, out):
    torch, capi, lib, _, _ = env
    B, S, H, D = q.shape
    st = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))  # noqa: E731
    rc = lib.b200_fa_fwd_fp16(cfg, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, k.shape[1], H, D,
                              st(q), st(k), st(v), st(out), 1.0 / math.sqrt(D), int(causal), None)
    assert rc == 0, lib.b200_last_error().decode()
    assert capi.device_status() == 0
    return out


def _sample_rows(S, seed, count):
    """Query rows to check: tile edges at both ends of the sequence plus seeded random ones."""
    fixed = [0, 127, 128, 255, 256, S - 257, S - 256, S - 129, S - 128, S - 1]
    rng = np.random.Generator(np.random.PCG64(seed))
    rows = set(r for r in fixed if 0 <= r < S) | set(int(r) for r in rng.choice(S, size=count, replace=False))
    return np.array(sorted(rows), dtype=np.int32)


def test_config5_attention_head_slice_of_full_tensors(env):
    """B=1 H=64 S=32768 D=128, seed 5: heads [24, 32) -- the slice of rank 3 of 8 -- read from
    and written into full [B,S,H,D] tensors through strides.  The other heads are NaN on input
    and must stay untouched on output."""
    torch, capi, lib, oracle, dev = env
    B, S, H, D, h0, hn = 1, 32768, 64, 128, 24, 8
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, hn, D, seed=5)
    rows = _sample_rows(S, 5, 8)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, False, rows=rows)
    full_in = []
    for bits in (q_bits, k_bits, v_bits):
        t = torch.full((B, S, H, D), float("nan"), dtype=torch.float16, device=dev)
        t[:, :, h0:h0 + hn] = torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.float16)
        full_in.append(t)
    q, k, v = (t[:, :, h0:h0 + hn] for t in full_in)
    sel = torch.from_numpy(rows).long().to(dev)
    for cfg in _layout_defaults(capi, D):
        o_full = torch.full((B, S, H, D), float("nan"), dtype=torch.float16, device=dev)
        _fa(env, cfg, q, k, v, False, o_full[:, :, h0:h0 + hn])
        got = o_full[:, :, h0:h0 + hn][:, sel].float().cpu().numpy()
        err = np.abs(got - ref).max()
        assert np.isfinite(err) and err <= ABS_BOUND, (capi.fa_configs()[cfg]["name"], err)
        rest = torch.cat([o_full[:, :, :h0], o_full[:, :, h0 + hn:]], dim=2)
        assert bool(torch.isnan(rest.float()).all()), "the head slice call wrote outside its heads"
        assert bool(torch.isfinite(o_full[:, :, h0:h0 + hn].float()).all())


# (seq_len, head_dim, head_num, batch): the entries of the reference list with seq_len >= 2048
LARGE_SHAPES = [(2048, 64, 16, 1), (2048, 64, 32, 8), (4096, 128, 32, 1), (4096, 128, 64, 2), (8192, 128, 32, 1),
                (8192, 128, 80, 4), (16384, 128, 32, 1)]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", LARGE_SHAPES, ids=lambda s: "s%d_d%d_h%d_b%d" % s)
def test_reference_shape_list_large_entries(env, shape, causal):
    """Inputs are drawn on the device (torch, seeded) and their bits copied back for the
    oracle, which checks tile-edge and random query rows of every (batch, head)."""
    torch, capi, lib, oracle, dev = env
    S, D, H, B = shape
    gen = torch.Generator(device=dev)
    gen.manual_seed(S + D + H + B)
    q, k, v = (torch.randn(B, S, H, D, device=dev, generator=gen).to(torch.float16) for _ in range(3))
    q_bits, k_bits, v_bits = (t.cpu().numpy().view(np.uint16) for t in (q, k, v))
    rows = _sample_rows(S, S + H, 6)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, causal, rows=rows)
    sel = torch.from_numpy(rows).long().to(dev)
    outs = []
    for cfg in _layout_defaults(capi, D):
        o = torch.full((B, S, H, D), float("nan"), dtype=torch.float16, device=dev)
        _fa(env, cfg, q, k, v, causal, o)
        err = np.abs(o[:, sel].float().cpu().numpy() - ref).max()
        assert np.isfinite(err) and err <= ABS_BOUND, (capi.fa_configs()[cfg]["name"], err)
        assert bool(torch.isfinite(o.float()).all())
        outs.append(o)
    # the layouts agree with each other everywhere, not only on the sampled rows
    for o in outs[1:]:
        assert (o.float() - outs[0].float()).abs().max().item() <= ABS_BOUND
