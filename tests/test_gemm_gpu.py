"""GPU parity tests of the BF16 GEMM, called through the C ABI (ctypes), checked against
the CPU oracle on the same seeded inputs.

Tolerances: the reference harness's rule |got-ref| <= 1e-2 + 5e-2*|ref| (gemm/test.cpp:29-30
of HugeOrca/sm120-dl) AND max |got-ref| / max(|ref|, rms(ref)) <= 1e-2 against the
fp64-accumulated host GEMM (the output is rounded to bf16: half an ulp is 2^-9 = 0.002
relative)."""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_BOUND = 1e-2


@pytest.fixture(scope="module")
def env(cuda_device, oracle):
    import torch
    from sm120_dl_b200 import capi
    return torch, capi, capi.lib(), oracle, cuda_device


def _to_dev(torch, bits, dev, dtype):
    return torch.from_numpy(bits.view(np.int16)).to(dev).view(dtype)


def _run(env, cfg, a, b, M, N, K, c=None, lda=None, ldb=None, ldc=None):
    torch, capi, lib, _, dev = env
    if c is None:
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)  # poison: every element must be written
    rc = lib.b200_gemm_bf16_tn(cfg, M, N, K, a.data_ptr(), lda or K, b.data_ptr(), ldb or K, c.data_ptr(),
                               ldc or N, None)
    assert rc == 0, lib.b200_last_error().decode()
    assert capi.device_status() == 0
    return c


def _check(oracle, got, ref):
    st = oracle.compare(got, ref, 1e-2, 5e-2)
    assert st["passed"], st
    assert st["max_rel_bounded"] <= REL_BOUND, st
    return st


def test_config1_512_cubed_uniform(env):
    """M=N=K=512, uniform[-1,1], seed 0: every config that divides the shape."""
    torch, capi, lib, oracle, dev = env
    a_bits, b_bits = oracle.make_gemm_inputs(512, 512, 512, 0, "uniform1")
    ref = oracle.gemm_f64(a_bits, b_bits)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    ran = 0
    for i, cfg in enumerate(capi.gemm_configs()):
        if 512 % cfg["bm"] or 512 % cfg["bn"]:
            continue
        c = _run(env, i, a, b, 512, 512, 512)
        _check(oracle, c.float().cpu().numpy(), ref)
        ran += 1
    assert ran >= 12


@pytest.mark.parametrize("kblocks", [1, 2, 7, 23])
def test_every_config_on_its_smallest_shapes(env, kblocks):
    """One tile and 2x3 tiles per config, with K from one k-block up (ring wrap-around)."""
    torch, capi, lib, oracle, dev = env
    for i, cfg in enumerate(capi.gemm_configs()):
        if cfg["split_k"] == 1 and cfg["bs_w"] != 8 and kblocks != 2:
            continue  # raster width changes tile order only; cover it once
        if kblocks < cfg["split_k"]:
            continue  # refused: fewer k-blocks than CTAs sharing the tile (tested below)
        for tm, tn in ((1, 1), (2, 3)):
            M, N, K = cfg["bm"] * tm, cfg["bn"] * tn, 64 * kblocks
            a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 100 + i, "uniform01")
            a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
            c = _run(env, i, a, b, M, N, K)
            _check(oracle, c.float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits))


def test_identity_b_reproduces_a_exactly(env):
    """B = I: C must equal A bit for bit (catches a wrong swizzle or lane mapping)."""
    torch, capi, lib, oracle, dev = env
    K = N = 512
    M = 768
    a_bits, _ = oracle.make_gemm_inputs(M, 8, K, 5, "uniform1")
    a = _to_dev(torch, a_bits, dev, torch.bfloat16)
    eye = torch.eye(N, K, dtype=torch.bfloat16, device=dev)
    for name in ("bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "bf16_bm128_bn128_bk64_s6_cta1_acc2_bsw8",
                 "bf16_bm256_bn64_bk64_s8_cta2_acc2_bsw8", "bf16_bm512_bn256_bk64_s4_cta2_acc2_bsw16"):
        c = _run(env, lib.b200_gemm_find_config(name.encode()), a, eye, M, N, K)
        assert torch.equal(c.view(torch.int16), a.view(torch.int16)), name


def test_deterministic_and_many_tiles_per_cta(env):
    """More tiles than CTAs (persistent loop + accumulator double buffering), run twice."""
    torch, capi, lib, oracle, dev = env
    M, N, K = 4096, 3072, 256
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 6)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    ref = oracle.gemm_f64(a_bits, b_bits)
    for name in ("bf16_bm128_bn64_bk64_s8_cta1_acc2_bsw8", "bf16_bm256_bn128_bk64_s8_cta2_acc2_bsw8"):
        idx = lib.b200_gemm_find_config(name.encode())
        c1 = _run(env, idx, a, b, M, N, K)
        c2 = _run(env, idx, a, b, M, N, K)
        assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))
        _check(oracle, c1.float().cpu().numpy(), ref)


@pytest.mark.parametrize("shape", [(8192, 3584, 192), (8062, 3600, 200), (1536, 520, 1096)])
def test_tall_tiles_two_accumulators_per_cta(env, shape):
    """512 x 256 tiles (two 128-row halves of A per CTA against one B block): up to four tiles
    per CTA pair, so both accumulators are reused and their barriers change phase; K shorter
    than the ring; ragged M, N and K; a column slab of a wider C; two destinations."""
    torch, capi, lib, oracle, dev = env
    M, N, K = shape
    lda = (K + 7) // 8 * 8
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, lda, 31)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    rows = min(M, 1200)
    ref = oracle.gemm_f64(a_bits[:, :K].copy(), b_bits[:, :K].copy(), row_begin=M - rows, row_count=rows)
    first = None
    for name in ("bf16_bm512_bn256_bk64_s4_cta2_acc2_bsw16", "bf16_bm512_bn256_bk64_s3_cta2_acc2_bsw12"):
        idx = lib.b200_gemm_find_config(name.encode())
        assert idx >= 0 and lib.b200_gemm_uses_stream_k(idx, M, N, K) == 0
        ldc = (N + 7) // 8 * 8 + 64
        wide = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device=dev)
        _run(env, idx, a, b, M, N, K, c=wide, lda=lda, ldb=lda, ldc=ldc)
        c = wide[:, :N]
        assert bool(torch.isnan(wide[:, N:].float()).all()), "wrote outside its column slab"
        _check(oracle, c[M - rows:].float().cpu().numpy(), ref)
        assert bool(torch.isfinite(c.float()).all())
        if first is None:
            first = c.clone()
        assert torch.equal(c.contiguous().view(torch.int16), first.contiguous().view(torch.int16)), name
        outs = [torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in outs])
        rc = lib.b200_gemm_bf16_tn_scatter(idx, M, N, K, a.data_ptr(), lda, b.data_ptr(), lda, ptrs, 2, ldc, None)
        assert rc == 0, lib.b200_last_error().decode()
        assert capi.device_status() == 0
        for t in outs:
            assert torch.equal(t[:, :N].contiguous().view(torch.int16), first.contiguous().view(torch.int16)), name
    # the 256 x 256 tile computes the same sums in the same order: bit-identical
    base = _run(env, lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8"), a, b, M, N, K,
                lda=lda, ldb=lda)
    assert torch.equal(base.view(torch.int16), first.contiguous().view(torch.int16))


def test_leading_dimensions_column_slab(env):
    """An N-shard writes its slab of a full-width C and reads a row slab of B."""
    torch, capi, lib, oracle, dev = env
    M, N, K = 512, 1024, 384
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 8)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    full = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    idx = lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8")
    for n0 in range(0, N, 256):
        _run(env, idx, a, b[n0:n0 + 256], M, 256, K, c=full[:, n0:n0 + 256], ldc=N)
    _check(oracle, full.float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits))
    # padded A (lda > K): the padding must not be read
    a_pad = torch.full((M, K + 64), float("nan"), dtype=torch.bfloat16, device=dev)
    a_pad[:, :K] = a
    c = _run(env, idx, a_pad, b, M, N, K, lda=K + 64)
    _check(oracle, c.float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits))


def test_config2_8192_cubed_rows_and_linearity(env):
    """M=N=K=8192, N(0,1)/sqrt(K), seed 1.  The oracle checks a seeded subset of rows (each
    output row depends on one row of A and all of B); a size-independent property covers
    the rest: the column sums of C equal (sum of A's rows) @ B^T."""
    torch, capi, lib, oracle, dev = env
    n = 8192
    a_bits, b_bits = oracle.make_gemm_inputs(n, n, n, 1)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    idx = lib.b200_gemm_default_config(n, n, n)
    assert lib.b200_gemm_get_config(idx).contents.cta_group == 2
    c = _run(env, idx, a, b, n, n, n)
    rng = np.random.Generator(np.random.PCG64(1))
    for r0 in sorted(rng.choice(n // 64, size=3, replace=False) * 64):
        ref = oracle.gemm_f64(a_bits, b_bits, row_begin=int(r0), row_count=64)
        _check(oracle, c[r0:r0 + 64].float().cpu().numpy(), ref)
    col_sums = c.double().sum(dim=0).cpu().numpy()
    a_sum = oracle.f32_from_bf16_bits(a_bits).astype(np.float64).sum(axis=0)
    expect = oracle.f32_from_bf16_bits(b_bits).astype(np.float64) @ a_sum
    # 8192 outputs per column, each off by at most half a bf16 ulp of a value of size ~1/sqrt(K)*...;
    # rounding errors are unbiased, so the sum stays within a few parts in 1e3 of the column scale
    assert np.abs(col_sums - expect).max() <= 2e-3 * np.sqrt(n) * c.float().abs().max().item()


@pytest.mark.parametrize("shape", [(300, 200, 100), (129, 264, 65), (1000, 72, 520), (1, 8, 8)])
def test_shapes_no_tile_divides(env, shape):
    """Ragged M, N and K (the reference refuses these; here TMA zero-fills and clips).  The
    rows are padded to a multiple of 8 elements and the padding is poisoned."""
    torch, capi, lib, oracle, dev = env
    M, N, K = shape
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 50 + M)
    ref = oracle.gemm_f64(a_bits, b_bits)
    lda = ldb = (K + 7) // 8 * 8
    ldc = (N + 7) // 8 * 8
    a = torch.full((M, lda), float("nan"), dtype=torch.bfloat16, device=dev)
    b = torch.full((N, ldb), float("nan"), dtype=torch.bfloat16, device=dev)
    a[:, :K] = _to_dev(torch, a_bits, dev, torch.bfloat16)
    b[:, :K] = _to_dev(torch, b_bits, dev, torch.bfloat16)
    for name in ("bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "bf16_bm128_bn64_bk64_s8_cta1_acc2_bsw8", None):
        idx = lib.b200_gemm_default_config(M, N, K) if name is None else lib.b200_gemm_find_config(name.encode())
        c = torch.full((M + 3, ldc), 7.0, dtype=torch.bfloat16, device=dev)
        _run(env, idx, a, b, M, N, K, c=c, lda=lda, ldb=ldb, ldc=ldc)
        _check(oracle, c[:M, :N].float().cpu().numpy(), ref)
        assert (c[M:] == 7.0).all() and (c[:, N:] == 7.0).all(), "stores leaked past the edge of C"


def test_error_paths(env):
    torch, capi, lib, oracle, dev = env
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device=dev)
    idx = lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8")
    assert lib.b200_gemm_bf16_tn(idx, 256, 0, 64, a.data_ptr(), 64, a.data_ptr(), 64, a.data_ptr(), 128, None) == -2
    assert b"must be positive" in lib.b200_last_error()
    assert lib.b200_gemm_bf16_tn(idx, 256, 128, 64, a.data_ptr(), 60, a.data_ptr(), 64, a.data_ptr(), 128, None) == -1
    assert lib.b200_gemm_bf16_tn(idx, 256, 132, 64, a.data_ptr(), 64, a.data_ptr(), 64, a.data_ptr(), 136, None) == -2
    assert b"multiple of 8" in lib.b200_last_error()
    # a base pointer that is not 16-byte aligned cannot be described to the TMA engine
    assert lib.b200_gemm_bf16_tn(idx, 256, 256, 64, a.data_ptr() + 2, 64, a.data_ptr(), 64, a.data_ptr(), 256, None) == -1
    assert b"aligned" in lib.b200_last_error()
    assert capi.device_status() == 0


def test_python_operator_and_streams(env):
    torch, capi, lib, oracle, dev = env
    from sm120_dl_b200 import ops
    a_bits, b_bits = oracle.make_gemm_inputs(256, 512, 128, 12)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        c = ops.gemm_bf16_tn(a, b)
    s.synchronize()
    _check(oracle, c.float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits))
    with pytest.raises(ValueError):
        ops.gemm_bf16_tn(a, b[:, :64])
    with pytest.raises(ValueError):
        ops.gemm_bf16_tn(a.float(), b)
    with pytest.raises(capi.B200Error):
        ops.gemm_bf16_tn(a, b[:100])          # N = 100 is not a multiple of 8
    c100 = ops.gemm_bf16_tn(a[:100], b)       # a ragged M is fine
    _check(oracle, c100.float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits)[:100])


def test_scatter_writes_every_destination(env):
    """The multi-destination epilogue (used to fuse the gather into the GEMM): two local
    windows of two different full-width matrices must both receive the product."""
    torch, capi, lib, oracle, dev = env
    from sm120_dl_b200 import ops
    M, N, K = 512, 512, 256
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 31)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    full = [torch.full((M, 3 * N), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(3)]
    outs = [full[0][:, N:2 * N], full[1][:, 0:N], full[2][:, 2 * N:3 * N]]
    ops.gemm_bf16_tn_scatter(a, b, outs)
    assert capi.device_status() == 0
    ref = oracle.gemm_f64(a_bits, b_bits)
    for t in outs:
        _check(oracle, t.float().cpu().numpy(), ref)
    assert torch.equal(outs[0].contiguous().view(torch.int16), outs[1].contiguous().view(torch.int16))
    # nothing outside the windows was touched
    assert torch.isnan(full[0][:, :N]).all() and torch.isnan(full[0][:, 2 * N:]).all()
    with pytest.raises(ValueError):
        ops.gemm_bf16_tn_scatter(a, b, [])
    ptrs = (ctypes.c_void_p * 9)(*[outs[0].data_ptr()] * 9)
    assert lib.b200_gemm_bf16_tn_scatter(0, 256, 256, 64, a.data_ptr(), 64, b.data_ptr(), 64, ptrs, 9, 256, None) == -1


def test_fp16_operands(env):
    """fp16 in / fp16 out through b200_gemm_f16_tn against numpy float64."""
    torch, capi, lib, oracle, dev = env
    from sm120_dl_b200 import ops
    M, N, K = 512, 768, 320
    rng = np.random.Generator(np.random.PCG64(61))
    a_h = rng.uniform(-1, 1, size=(M, K)).astype(np.float16)
    b_h = rng.uniform(-1, 1, size=(N, K)).astype(np.float16)
    ref = a_h.astype(np.float64) @ b_h.astype(np.float64).T
    a, b = torch.from_numpy(a_h).to(dev), torch.from_numpy(b_h).to(dev)
    for cfg in ("bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "bf16_bm128_bn128_bk64_s6_cta1_acc2_bsw8",
                "bf16_bm512_bn256_bk64_s4_cta2_acc2_bsw16"):
        c = ops.gemm_f16_tn(a, b, config=cfg)
        assert capi.device_status() == 0
        st = oracle.compare(c.float().cpu().numpy(), ref, 1e-2, 5e-2)
        # fp16 output: half an ulp is 2^-11, far inside the bounded relative error of 1e-2
        assert st["passed"] and st["max_rel_bounded"] <= 2e-3, st
    with pytest.raises(ValueError):
        ops.gemm_f16_tn(a.bfloat16(), b)


def test_split_k_skinny_shape_and_refusals(env):
    """M=128 with a long K (a shape of the reference's list, gemm/test.cpp:38-61): the default
    choice is a split-K config, every split-K config matches the fp64 oracle, runs are
    bit-reproducible, and a K with fewer k-blocks than the split is refused."""
    torch, capi, lib, oracle, dev = env
    M, N, K = 128, 4096, 14336
    cfgs = capi.gemm_configs()
    assert cfgs[lib.b200_gemm_default_config(M, N, K)]["split_k"] > 1
    assert cfgs[lib.b200_gemm_default_config(8192, 8192, 8192)]["split_k"] == 1
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 21)
    ref = oracle.gemm_f64(a_bits, b_bits)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    ran = 0
    for i, cfg in enumerate(cfgs):
        if cfg["split_k"] == 1:
            continue
        c1 = _run(env, i, a, b, M, N, K)
        c2 = _run(env, i, a, b, M, N, K)
        assert torch.equal(c1.view(torch.int16), c2.view(torch.int16)), cfg["name"]
        _check(oracle, c1.float().cpu().numpy(), ref)
        ran += 1
        # 3 k-blocks cannot be shared by 4 or 8 CTAs
        if cfg["split_k"] > 3:
            out = torch.empty((M, 64), dtype=torch.bfloat16, device=dev)
            rc = lib.b200_gemm_bf16_tn(i, M, 64, 192, a.data_ptr(), K, b.data_ptr(), K, out.data_ptr(), 64, None)
            assert rc == -2 and b"fewer 64-element blocks" in lib.b200_last_error()
    assert ran == 9


def test_split_k_ragged_shape_fp16_and_two_destinations(env):
    """Split-K on a shape no tile divides, in fp16, and stored to two outputs at once."""
    torch, capi, lib, oracle, dev = env
    from sm120_dl_b200 import ops
    M, N, K = 100, 200, 1096 + 8
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 22)
    ref = oracle.gemm_f64(a_bits, b_bits)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    for name in ("bf16_bm128_bn64_bk64_s8_cta1_splitk4", "bf16_bm128_bn128_bk64_s6_cta1_splitk8"):
        outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ops.gemm_bf16_tn_scatter(a, b, outs, config=name)
        torch.cuda.synchronize()
        assert capi.device_status() == 0
        assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
        _check(oracle, outs[0].float().cpu().numpy(), ref)
        ah, bh = a.float().half(), b.float().half()
        ch = ops.gemm_f16_tn(ah, bh, config=name)
        torch.cuda.synchronize()
        want = (ah.double() @ bh.double().T)
        assert (ch.double() - want).abs().max().item() <= 2e-3 * max(1.0, want.abs().max().item())


def test_split_k_leading_dimensions_several_row_tiles_ragged_k(env):
    """Split-K with padded operands (lda, ldb > K), a column slab of a wider C (ldc > N),
    several row tiles, an N no tile divides and a K that ends inside a k-block."""
    torch, capi, lib, oracle, dev = env
    M, N, K = 320, 200, 2048 + 24
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 23)
    ref = oracle.gemm_f64(a_bits, b_bits)
    a_pad = torch.full((M, K + 8), float("nan"), dtype=torch.bfloat16, device=dev)
    b_pad = torch.full((N, K + 16), float("nan"), dtype=torch.bfloat16, device=dev)
    a_pad[:, :K] = _to_dev(torch, a_bits, dev, torch.bfloat16)
    b_pad[:, :K] = _to_dev(torch, b_bits, dev, torch.bfloat16)
    for name in ("bf16_bm128_bn64_bk64_s8_cta1_splitk2", "bf16_bm128_bn128_bk64_s6_cta1_splitk4",
                 "bf16_bm128_bn256_bk64_s4_cta1_splitk8"):
        wide = torch.full((M, 512), -7.0, dtype=torch.bfloat16, device=dev)
        idx = lib.b200_gemm_find_config(name.encode())
        assert idx >= 0, name
        _run(env, idx, a_pad, b_pad, M, N, K, c=wide[:, 104:104 + N], lda=K + 8, ldb=K + 16, ldc=512)
        _check(oracle, wide[:, 104:104 + N].float().cpu().numpy(), ref)
        # nothing outside the slab was touched
        assert bool((wide[:, :104] == -7.0).all()) and bool((wide[:, 104 + N:] == -7.0).all()), name


@pytest.fixture
def stream_k(env):
    """Stream-K switched on for one test (it is off by default), and off again afterwards."""
    lib = env[2]
    assert lib.b200_gemm_set_stream_k(1) == 0
    yield
    assert lib.b200_gemm_set_stream_k(0) == 0


def test_stream_k_is_off_by_default(env):
    torch, capi, lib, oracle, dev = env
    idx = lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8")
    assert lib.b200_gemm_uses_stream_k(idx, 2560, 2560, 2048) == 0
    assert lib.b200_gemm_set_stream_k(2) == -1
    assert lib.b200_gemm_set_stream_k(1) == 0
    assert lib.b200_gemm_uses_stream_k(idx, 2560, 2560, 2048) == 1
    assert lib.b200_gemm_uses_stream_k(idx, 2560, 2560, 512) == 0     # 8 k-blocks: too short to pay
    assert lib.b200_gemm_set_stream_k(0) == 0


@pytest.mark.parametrize("shape", [(2560, 2560, 1024), (1280, 2560, 2048), (2500, 2440, 1096), (16384, 512, 4096)],
                         ids=lambda s: "%dx%dx%d" % s)
def test_ragged_last_wave_is_cut_along_k(env, stream_k, shape):
    """Shapes whose tiles do not fill the last wave, with stream-K on: the launcher splits the
    tail tiles' k-blocks over all CTA groups, partial sums go through a workspace and are added
    in a fixed order.  Every element against the oracle, run-to-run bitwise equality, for
    CTA-pair and single-CTA configs, and through the multi-destination entry point."""
    torch, capi, lib, oracle, dev = env
    M, N, K = shape
    a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 11)
    a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
    rows = min(M, 2560)
    ref = oracle.gemm_f64(a_bits, b_bits, row_begin=M - rows, row_count=rows)
    cut = 0
    for name in ("bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8", "bf16_bm128_bn256_bk64_s4_cta1_acc2_bsw8",
                 "bf16_bm256_bn128_bk64_s8_cta2_acc2_bsw8"):
        idx = lib.b200_gemm_find_config(name.encode())
        assert idx >= 0
        cut += lib.b200_gemm_uses_stream_k(idx, M, N, K)
        c = _run(env, idx, a, b, M, N, K)
        _check(oracle, c[M - rows:].float().cpu().numpy(), ref)
        assert bool(torch.isfinite(c.float()).all())
        again = _run(env, idx, a, b, M, N, K)
        assert torch.equal(c.view(torch.int16), again.view(torch.int16)), name
        # two destinations at once
        outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in outs])
        rc = lib.b200_gemm_bf16_tn_scatter(idx, M, N, K, a.data_ptr(), K, b.data_ptr(), K, ptrs, 2, N, None)
        assert rc == 0, lib.b200_last_error().decode()
        assert capi.device_status() == 0
        for t in outs:
            assert torch.equal(t.view(torch.int16), c.view(torch.int16)), name
    assert cut >= 1, "none of the configs cut this shape's last wave: the test shape no longer exercises stream-K"


def test_stream_k_overlapping_streams(env, stream_k):
    """Launches on two streams at once: every launch has its own stream-ordered workspace."""
    torch, capi, lib, oracle, dev = env
    M, N, K = 2560, 2560, 2048
    idx = lib.b200_gemm_find_config(b"bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8")
    assert lib.b200_gemm_uses_stream_k(idx, M, N, K) == 1
    streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
    problems = []
    for i, st in enumerate(streams):
        a_bits, b_bits = oracle.make_gemm_inputs(M, N, K, 20 + i)
        a, b = _to_dev(torch, a_bits, dev, torch.bfloat16), _to_dev(torch, b_bits, dev, torch.bfloat16)
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        problems.append((a_bits, b_bits, a, b, c))
    torch.cuda.synchronize()
    for rep in range(6):
        for (a_bits, b_bits, a, b, c), st in zip(problems, streams):
            rc = lib.b200_gemm_bf16_tn(idx, M, N, K, a.data_ptr(), K, b.data_ptr(), K, c.data_ptr(), N,
                                       ctypes.c_void_p(st.cuda_stream))
            assert rc == 0, lib.b200_last_error().decode()
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for a_bits, b_bits, a, b, c in problems:
        _check(oracle, c[:256].float().cpu().numpy(), oracle.gemm_f64(a_bits, b_bits, row_begin=0, row_count=256))
