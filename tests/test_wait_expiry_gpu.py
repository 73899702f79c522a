"""GPU test of the bounded waits: a wait that cannot succeed gives up, the kernel returns, the
status word says where, and the library keeps working.  The failing condition is a barrier
whose announced bytes never arrive (nothing faults, traps or spins without a limit); the
wait limit is 5 ms for this call instead of the kernels' 2 s."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_the_library_stays_usable(cuda_device, oracle):
    import torch
    from sm120_dl_b200 import capi, ops

    lib = capi.lib()
    assert capi.device_status() == 0
    assert lib.b200_selftest_wait_expiry(5, None) == 0, lib.b200_last_error().decode()
    torch.cuda.synchronize()                      # the kernel returned; no sticky CUDA error
    code = capi.device_status()
    assert code == 0x80007E57, hex(code)          # the consumer's wait site
    assert capi.device_status() == 0              # reading cleared it

    # bad arguments are refused on the host
    assert lib.b200_selftest_wait_expiry(0, None) == -1
    assert lib.b200_selftest_wait_expiry(5000, None) == -1

    # a normal GEMM afterwards is correct
    a_bits, b_bits = oracle.make_gemm_inputs(256, 256, 256, seed=9)
    a = torch.from_numpy(a_bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    c = ops.gemm_bf16_tn(a, b)
    assert capi.device_status() == 0
    st = oracle.compare(c.float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits), 1e-2, 5e-2)
    assert st["passed"] and st["max_rel_bounded"] <= 1e-2, st
