"""GPU test of b200_gemm_bf16_tn_noalloc, the GEMM entry point for callers that are not
allowed to allocate device memory (a process whose GPU memory is already owned by a
framework's pool, a service with a fixed memory budget, a latency-critical loop).  It must
give the same C as b200_gemm_bf16_tn while taking its scratch from an array built into the
library instead of cudaMalloc.

The file name sorts last on purpose: a run that stops at the first failure has then
already run every other test.  The test passes on its own in a fresh process (the new
entry point is called first, so its one-time set-up cannot lean on the other entry
point's) and after the rest of the suite.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_matches_allocating_entry_point_twice(cuda_device, oracle):
    import torch
    from sm120_dl_b200 import capi

    lib = capi.lib()
    M, N, K = 1024, 768, 512
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, seed=77)
    a = torch.from_numpy(a_bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    ref = oracle.gemm_f64(a_bits, b_bits)
    cfg = lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8")
    assert cfg >= 0

    # Everything the calls need exists before them; from here on only the entry points run.
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device) for _ in range(3)]
    torch.cuda.synchronize()

    def noalloc(c):
        rc = lib.b200_gemm_bf16_tn_noalloc(cfg, M, N, K, a.data_ptr(), K, b.data_ptr(), K, c.data_ptr(), N, None)
        assert rc == 0, lib.b200_last_error().decode()

    # The first call on a device does the one-time set-up (symbol address, device
    # attributes, the kernel's shared-memory attribute; the CUDA runtime may load the
    # kernel image then).  From the second call on, the free device memory must not move:
    # that is the property this entry point exists for.
    noalloc(outs[0])
    assert capi.noalloc_status() == 0
    free_before, _ = torch.cuda.mem_get_info()
    # two calls in a row (each finds the scratch array as the previous one left it)
    for c in outs[:2]:
        noalloc(c)
    assert capi.noalloc_status() == 0, "a bounded wait gave up in the allocation-free launch"
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes across noalloc calls"

    rc = lib.b200_gemm_bf16_tn(cfg, M, N, K, a.data_ptr(), K, b.data_ptr(), K, outs[2].data_ptr(), N, None)
    assert rc == 0, lib.b200_last_error().decode()
    assert capi.device_status() == 0

    want = outs[2].float().cpu().numpy()
    for c in outs[:2]:
        got = c.float().cpu().numpy()
        # same kernel, same inputs: the suite's GEMM tolerance (|d| <= 1e-2 + 5e-2 |ref|,
        # bounded relative error <= 1e-2) against both the other entry point and the oracle
        st = oracle.compare(got, want, 1e-2, 5e-2)
        assert st["passed"] and st["max_rel_bounded"] <= 1e-2, st
        st = oracle.compare(got, ref, 1e-2, 5e-2)
        assert st["passed"] and st["max_rel_bounded"] <= 1e-2, st
        # and, the kernel being deterministic, bit for bit what the allocating entry point gives
        assert torch.equal(c.view(torch.int16), outs[2].view(torch.int16))


def test_noalloc_rejects_bad_arguments(cuda_device):
    import torch
    from sm120_dl_b200 import capi

    lib = capi.lib()
    x = torch.zeros(256, 256, dtype=torch.bfloat16, device=cuda_device)
    cfg = lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8")
    assert lib.b200_gemm_bf16_tn_noalloc(cfg, 0, 256, 256, x.data_ptr(), 256, x.data_ptr(), 256, x.data_ptr(), 256, None) == -2
    assert b"must be positive" in lib.b200_last_error()
    assert lib.b200_gemm_bf16_tn_noalloc(-1, 256, 256, 256, x.data_ptr(), 256, x.data_ptr(), 256, x.data_ptr(), 256, None) == -1
    assert lib.b200_gemm_bf16_tn_noalloc(cfg, 256, 256, 256, None, 256, x.data_ptr(), 256, x.data_ptr(), 256, None) == -1
