"""GPU parity tests of the FP16 attention forward, called through the C ABI (ctypes) and
through the flashatten_v3_sm120 module, checked against the CPU oracle (fp32
softmax(Q K^T * scale) V) on the same seeded inputs.

Tolerance: max |got - ref| <= 2e-3 absolute for N(0,1) inputs; additionally the
reference script's rule |got-ref| <= 0.075 + 0.075*|ref| (verify.py:15-16, 64-80 of
HugeOrca/sm120-dl) on its own input scale (randn * 0.5)."""

import ctypes
import math
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ABS_BOUND = 2e-3
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def env(cuda_device, oracle):
    import torch
    from sm120_dl_b200 import capi
    return torch, capi, capi.lib(), oracle, cuda_device


def _dev(torch, bits, dev):
    return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.float16)


def _fwd(env, cfg, q, k, v, causal, out=None):
    torch, capi, lib, _, dev = env
    B, S, H, D = q.shape
    if out is None:
        out = torch.full((B, S, H, D), float("nan"), dtype=torch.float16, device=dev)
    st = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))  # noqa: E731
    rc = lib.b200_fa_fwd_fp16(cfg, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, k.shape[1], H, D,
                              st(q), st(k), st(v), st(out), 1.0 / math.sqrt(D), int(causal), None)
    assert rc == 0, lib.b200_last_error().decode()
    assert capi.device_status() == 0
    return out


def _layout_defaults(capi, head_dim):
    """Index of the first config of every softmax layout for this head_dim (the first of them
    is the library's default for the head_dim)."""
    first = {}
    for i, cfg in enumerate(capi.fa_configs()):
        if cfg["head_dim"] == head_dim:
            first.setdefault(cfg["softmax_layout"], i)
    return sorted(first.values())


# seq_len, head_dim, head_num, batch: the small entries of the reference's shape list
# (verify.py:26-45) plus sizes that cross tile boundaries
SMALL_SHAPES = [(64, 64, 1, 1), (128, 64, 1, 2), (192, 64, 4, 1), (256, 64, 8, 2), (128, 128, 4, 2),
                (256, 128, 4, 1), (320, 128, 3, 1), (448, 64, 5, 1), (1024, 128, 2, 1), (1088, 64, 2, 1)]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SMALL_SHAPES, ids=lambda s: "s%d_d%d_h%d_b%d" % s)
def test_small_shapes_every_config(env, shape, causal):
    torch, capi, lib, oracle, dev = env
    S, D, H, B = shape
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=S + D + H + B + int(causal))
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, causal)
    q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
    for i, cfg in enumerate(capi.fa_configs()):
        if cfg["head_dim"] != D:
            continue
        o = _fwd(env, i, q, k, v, causal)
        err = np.abs(o.float().cpu().numpy() - ref).max()
        assert np.isfinite(err) and err <= ABS_BOUND, (cfg["name"], err)


def test_config3_b4_h32_s4096_d128(env):
    """B=4 H=32 S=4096 D=128, N(0,1), seed 2.  The oracle checks a seeded subset of query
    rows of every (batch, head) (a row depends on all of K and V of its head and nothing
    else); row sums of softmax being 1 gives a size-independent check on all rows: with
    V = 1 every output is exactly 1."""
    torch, capi, lib, oracle, dev = env
    B, S, H, D = 4, 4096, 32, 128
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=2)
    q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
    rows = np.sort(np.random.Generator(np.random.PCG64(2)).choice(S, size=24, replace=False)).astype(np.int32)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, False, rows=rows)
    ones = torch.ones_like(v)
    assert lib.b200_fa_default_config(D) in _layout_defaults(capi, D)
    for idx in _layout_defaults(capi, D):
        o = _fwd(env, idx, q, k, v, False)
        err = np.abs(o[:, torch.from_numpy(rows).long().to(dev)].float().cpu().numpy() - ref).max()
        assert err <= ABS_BOUND, (capi.fa_configs()[idx]["name"], err)
        o1 = _fwd(env, idx, q, k, ones, False)
        assert (o1.float() - 1.0).abs().max().item() <= 2e-3
        # deterministic
        assert torch.equal(o.view(torch.int16), _fwd(env, idx, q, k, v, False).view(torch.int16))


def test_config4_b16_h32_s2048_d64(env):
    torch, capi, lib, oracle, dev = env
    B, S, H, D = 16, 2048, 32, 64
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=3)
    q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
    rows = np.sort(np.random.Generator(np.random.PCG64(3)).choice(S, size=12, replace=False)).astype(np.int32)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, False, rows=rows)
    for idx in _layout_defaults(capi, D):
        o = _fwd(env, idx, q, k, v, False)
        err = np.abs(o[:, torch.from_numpy(rows).long().to(dev)].float().cpu().numpy() - ref).max()
        assert err <= ABS_BOUND, (capi.fa_configs()[idx]["name"], err)


def test_head_slices_through_strides(env):
    """A head shard reads and writes slices of full [B,S,H,D] tensors."""
    torch, capi, lib, oracle, dev = env
    B, S, H, D = 2, 384, 6, 128
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=21)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, True)
    q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
    for idx in _layout_defaults(capi, D):
        full = torch.full((B, S, H, D), float("nan"), dtype=torch.float16, device=dev)
        for h0 in range(0, H, 2):
            _fwd(env, idx, q[:, :, h0:h0 + 2], k[:, :, h0:h0 + 2], v[:, :, h0:h0 + 2], True, out=full[:, :, h0:h0 + 2])
        assert np.abs(full.float().cpu().numpy() - ref).max() <= ABS_BOUND


def test_large_scores_do_not_overflow(env):
    """Scores far above the fp16 range of exp: the running-max rescale must keep P <= 2^8."""
    torch, capi, lib, oracle, dev = env
    B, S, H, D = 1, 512, 2, 64
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=33, std=6.0)
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, False)
    q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
    for idx in _layout_defaults(capi, D):
        o = _fwd(env, idx, q, k, v, False)
        err = np.abs(o.float().cpu().numpy() - ref).max()
        # outputs are O(6) here; fp16 output rounding alone is 2^-11 * 8
        assert np.isfinite(err) and err <= 2e-2, (capi.fa_configs()[idx]["name"], err)


def test_error_paths(env):
    torch, capi, lib, oracle, dev = env
    q = torch.zeros(1, 100, 1, 64, dtype=torch.float16, device=dev)
    st = (ctypes.c_int64 * 3)(6400, 64, 64)
    idx = lib.b200_fa_default_config(64)
    assert lib.b200_fa_fwd_fp16(idx, q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 1, 100, 100, 1, 64,
                                st, st, st, st, 0.125, 0, None) == -2
    assert b"multiple of 64" in lib.b200_last_error()
    assert capi.device_status() == 0


@pytest.fixture(scope="module")
def module(cuda_device):
    from sm120_dl_b200 import build
    build.build_lib()
    build.build_fa_module()
    sys.path.insert(0, os.path.join(ROOT, "sm120_dl_b200", "flashattention", "pybind", "build"))
    import flashatten_v3_sm120
    return flashatten_v3_sm120


def test_module_interface_and_reference_tolerance(env, module):
    """The calls verify.py makes, with its inputs (randn * 0.5) and its tolerance."""
    torch, capi, lib, oracle, dev = env
    assert module.default_config_name() == module.configs()[0][0]
    assert all(len(c) == 7 for c in module.configs())
    assert [64, 64, 1, 1] in [list(s) for s in module.supported_shapes()] and len(module.supported_shapes()) == 18
    for (S, D, H, B) in [(64, 64, 1, 1), (192, 64, 4, 1), (256, 128, 4, 1), (2048, 64, 16, 1)]:
        for causal in (False, True):
            q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=20260614 + S + D + H + B + int(causal), std=0.5)
            q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
            got = module.fwd(q, k, v, causal)
            assert got.shape == q.shape and got.dtype == torch.float16 and got.is_contiguous()
            rows = None if S <= 256 else np.arange(0, S, 64, dtype=np.int32)
            ref = oracle.attention_f32(q_bits, k_bits, v_bits, causal, rows=rows)
            g = got.float().cpu().numpy() if rows is None else got.float().cpu().numpy()[:, rows]
            assert oracle.compare(g, ref, 0.075, 0.075)["passed"]
            assert np.abs(g - ref).max() <= ABS_BOUND
            name = module.configs()[-1][0] if D == 128 else module.configs()[0][0]
            again = module.fwd_config(name, q, k, v, causal)
            assert np.abs(again.float().cpu().numpy() - got.float().cpu().numpy()).max() <= 1e-3


def test_module_rejections(env, module):
    torch, capi, lib, oracle, dev = env
    q = torch.zeros(1, 128, 2, 64, dtype=torch.float16, device=dev)
    with pytest.raises(RuntimeError, match="unknown flash_fwd config"):
        module.fwd_config("hd64_nope", q, q, q, False)
    with pytest.raises(RuntimeError, match="must use torch.float16"):
        module.fwd(q.float(), q, q)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        module.fwd(q.cpu(), q, q)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        module.fwd(q.transpose(1, 2), q, q)
    with pytest.raises(RuntimeError, match="k shape must match q shape"):
        module.fwd(q, q[:, :64].contiguous(), q)
    with pytest.raises(RuntimeError, match="seq_len must be a multiple of 64"):
        z = torch.zeros(1, 100, 2, 64, dtype=torch.float16, device=dev)
        module.fwd(z, z, z)
    with pytest.raises(RuntimeError, match="no flash_fwd config was built for head_dim=96"):
        z = torch.zeros(1, 128, 2, 96, dtype=torch.float16, device=dev)
        module.fwd(z, z, z)
    with pytest.raises(RuntimeError, match="expects head_dim=64"):
        z = torch.zeros(1, 128, 2, 128, dtype=torch.float16, device=dev)
        module.fwd_config(module.configs()[0][0], z, z, z)


def test_scatter_writes_every_destination(env):
    """The multi-destination epilogue (used to fuse the head gather into the kernel)."""
    torch, capi, lib, oracle, dev = env
    from sm120_dl_b200 import ops
    B, S, H, D = 1, 320, 2, 128
    q_bits, k_bits, v_bits = oracle.make_fa_inputs(B, S, H, D, seed=41)
    q, k, v = (_dev(torch, x, dev) for x in (q_bits, k_bits, v_bits))
    full = [torch.full((B, S, 6, D), float("nan"), dtype=torch.float16, device=dev) for _ in range(2)]
    outs = [full[0][:, :, 2:4], full[1][:, :, 2:4]]
    ops.flash_attn_fwd_scatter(q, k, v, outs, causal=True)
    assert capi.device_status() == 0
    ref = oracle.attention_f32(q_bits, k_bits, v_bits, True)
    for t in outs:
        assert np.abs(t.float().cpu().numpy() - ref).max() <= ABS_BOUND
    assert torch.isnan(full[0][:, :, :2]).all() and torch.isnan(full[1][:, :, 4:]).all()
    with pytest.raises(ValueError):  # destinations of different shapes
        ops.flash_attn_fwd_scatter(q, k, v, [full[0][:, :, 0:2], full[1][:, ::2, 0:2]])
