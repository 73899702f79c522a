"""The reference project's own kernels (its sources, rebuilt for sm_100a into
oracle/_ref/ by oracle/build_ref.py) as a same-box witness: fed the same seeded inputs as
the kernels of this library, both must be within the suite's tolerance of the CPU oracle
and of each other.  Skipped when the witness library has not been built (it needs a
checkout of the reference beside this repository)."""

import importlib.util
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location("ref_witness", os.path.join(ROOT, "oracle", "ref_witness.py"))
ref_witness = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(ref_witness)

needs_witness = pytest.mark.skipif(not ref_witness.available(), reason="oracle/_ref/libsm120ref.so not built")


@needs_witness
@pytest.mark.parametrize("shape", [(512, 512, 512), (1024, 768, 2048), (4096, 4096, 4096)], ids=lambda s: "%dx%dx%d" % s)
def test_gemm_reference_kernel_oracle_and_ours_agree(cuda_device, oracle, shape):
    import torch
    from sm120_dl_b200 import capi, ops

    M, N, K = shape
    dist = "uniform1" if shape == (512, 512, 512) else "normal_over_sqrt_k"
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 0 if dist == "uniform1" else 1, dist)
    a = torch.from_numpy(a_bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    rows = min(M, 256)
    ref = oracle.gemm_f64(a_bits, b_bits, row_begin=0, row_count=rows)
    ours = ops.gemm_bf16_tn(a, b)
    assert capi.device_status() == 0
    for which in ref_witness.GEMM_CONFIGS:
        theirs = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        ref_witness.gemm(which, a, b, theirs)
        torch.cuda.synchronize()
        for got in (theirs, ours):
            st = oracle.compare(got[:rows].float().cpu().numpy(), ref, 1e-2, 5e-2)
            assert st["passed"] and st["max_rel_bounded"] <= 1e-2, (which, st)
        # both round an fp32 accumulation of the same products to bf16: they differ by at most
        # one rounding step of the larger magnitude
        st = oracle.compare(ours.float().cpu().numpy(), theirs.float().cpu().numpy().astype(np.float64), 1e-2, 5e-2)
        assert st["passed"] and st["max_rel_bounded"] <= 1e-2, (which, st)


@needs_witness
@pytest.mark.parametrize("std", [0.5, 1.0])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(512, 128, 4, 2), (1024, 64, 4, 1), (2048, 128, 32, 1), (2048, 64, 32, 2)],
                         ids=lambda s: "s%d_d%d_h%d_b%d" % s)
def test_attention_reference_kernel_oracle_and_ours_agree(cuda_device, oracle, shape, causal, std):
    """std 0.5 is the input scale of the reference's own scripts (verify.py:58-60: randn * 0.5);
    there its kernel is within 5e-3 of the fp32 oracle.  On N(0,1) inputs (the benchmark
    configurations' scale) its non-causal head_dim-128 path was observed 0.075 and more away
    from the oracle on a B200, on isolated elements that differ from run to run, so for std 1.0
    the reference kernel is held to the reference's own rule |d| <= 0.075 + 0.075 |ref|
    (verify.py:15-16) on all but one element in a thousand.  The kernels of this library are
    held to 2e-3 on every element in both cases."""
    import torch
    from sm120_dl_b200 import capi, ops

    S, D, H, B = shape
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=S + D + H + B + int(causal), std=std)
    rows = np.unique(np.concatenate([np.arange(0, S, max(1, S // 24)), [S - 1]])).astype(np.int32)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, causal, rows=rows)
    q, k, v = (torch.from_numpy(x.view(np.int16)).to(cuda_device).view(torch.float16) for x in (q_bits, k_bits, v_bits))
    theirs = torch.full((B, S, H, D), float("nan"), dtype=torch.float16, device=cuda_device)
    ref_witness.attention(q, k, v, theirs, causal)
    torch.cuda.synchronize()
    sel = torch.from_numpy(rows).long().to(cuda_device)
    got_theirs = theirs[:, sel].float().cpu().numpy()
    assert np.isfinite(got_theirs).all()
    if std == 0.5:
        assert np.abs(got_theirs - ref).max() <= 5e-3
    else:
        outside = np.abs(got_theirs - ref) > 0.075 + 0.075 * np.abs(ref)
        assert outside.mean() <= 1e-3, (outside.sum(), np.abs(got_theirs - ref).max())
    first = {}
    for i, cfg in enumerate(capi.fa_configs()):
        if cfg["head_dim"] == D:
            first.setdefault(cfg["softmax_layout"], i)
    for idx in sorted(first.values()):
        ours = ops.flash_attn_fwd(q, k, v, causal=causal, config=idx)
        assert capi.device_status() == 0
        err = np.abs(ours[:, sel].float().cpu().numpy() - ref).max()
        assert np.isfinite(err) and err <= 2e-3, (capi.fa_configs()[idx]["name"], err)
        # the two GPU kernels against each other, on every element
        d = (ours.float() - theirs.float()).abs()
        if std == 0.5:
            assert d.max().item() <= 5e-3
        else:
            outside = d > 0.075 + 0.075 * ours.float().abs()
            assert outside.float().mean().item() <= 1e-3, (int(outside.sum()), d.max().item())
