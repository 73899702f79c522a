"""CPU tests of the host side: the config generators, the C ABI library's exports against
include/b200dl.h, config lookup, shard arithmetic and the multi-process gather logic
(gloo, world_size 2).  No kernel is launched here."""

import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sm120_dl_b200")


def _import_from(path, name):
    sys.path.insert(0, path)
    try:
        return __import__(name)
    finally:
        sys.path.remove(path)


@pytest.fixture(scope="module")
def lib():
    from sm120_dl_b200 import build, capi
    build.build_lib()
    return capi.lib()


# ----------------------------------------------------------------------- generators
def test_gemm_generator_rules():
    g = _import_from(os.path.join(PKG, "gemm"), "gemm_configs")
    cfgs = g.generate_configs(227)
    names = [c[0] for c in cfgs]
    assert len(names) == len(set(names)) and g.DEFAULT_NAME in names
    for name, bn, stages, cta_group, acc_bufs, bs_w in cfgs:
        assert g.smem_bytes(bn, stages, cta_group, acc_bufs) <= 227 * 1024
        assert bn * acc_bufs <= 512 and bn % 64 == 0 and cta_group in (1, 2)
        assert name == g.config_name(bn, stages, cta_group, acc_bufs, bs_w)
    # the budgets bite: 7 stages of a CTA-pair 256-wide tile do not fit, 64 KiB fits nothing big
    assert not g.is_valid_config(256, 7, 2, 2, 8, 227 * 1024)
    assert not g.is_valid_config(256, 3, 1, 3, 8, 227 * 1024)      # 768 tensor-memory columns
    assert not g.is_valid_config(200, 3, 1, 1, 8, 227 * 1024)      # N not a multiple of 64
    assert all(c[1] <= 64 for c in g.generate_configs(64))
    assert len(g.generate_configs(227, full=True)) > len(cfgs)
    # tall tiles: two accumulators of 256 columns, 48 KiB per stage; 5 stages do not fit
    tall = g.generate_tall_configs(227)
    assert {(c[1], c[2]) for c in tall} == {(256, 3), (256, 4)} and {c[3] for c in tall} == set(g.TALL_BS_W_VALUES)
    for name, bn, stages, bs_w in tall:
        assert name == g.tall_config_name(bn, stages, bs_w) and name.startswith("bf16_bm512_")
        assert g.tall_smem_bytes(bn, stages) <= 227 * 1024 and 2 * bn <= 512
    assert g.tall_smem_bytes(256, 5) > 227 * 1024 and not g.generate_tall_configs(100)


def test_gemm_generator_writes_reference_style_cmake(tmp_path):
    g = _import_from(os.path.join(PKG, "gemm"), "gemm_configs")
    out = tmp_path / "configs.cmake"
    inc = tmp_path / "g.inc"
    reg = tmp_path / "r.inc"
    cfgs = g.main(["--output", str(out), "--inc", str(inc), "--registry", str(reg), "--max-smem-kb", "200"])
    text = out.read_text()
    assert "set(GEMM_TN_MAX_SMEM_BYTES 204800)" in text and "set(GEMM_TN_CONFIGS" in text
    assert "set(GEMM_TN_DEFAULT_CONFIG" in text
    splitk = g.generate_splitk_configs(200)
    assert inc.read_text().count("B200_GEMM_CONFIG(\"") == len(cfgs)
    tall = g.generate_tall_configs(200)
    assert inc.read_text().count("B200_GEMM_SPLITK_CONFIG(\"") == len(splitk) == 9
    assert inc.read_text().count("B200_GEMM_TALL_CONFIG(\"") == len(tall) == 3     # 4 stages need > 200 KiB
    assert reg.read_text().count("B200_GEMM_ENTRY(") == len(cfgs) + len(splitk) + len(tall) + 1  # + the comment line
    for name, bn, stages, split_k in splitk:
        assert name == g.splitk_config_name(bn, stages, split_k) and split_k in (2, 4, 8)
        assert g.splitk_smem_bytes(bn, stages) <= 200 * 1024
        assert stages * g.stage_bytes(bn, 1) >= 128 * bn * 4   # the fp32 partial tile reuses the ring


def test_flash_generator_rules(monkeypatch, tmp_path):
    f = _import_from(os.path.join(PKG, "flashattention"), "flash_configs")
    cfgs = f.generate_configs(227)
    assert {c[1] for c in cfgs} == {64, 128}
    assert {c[4] for c in cfgs} == {1, 2, 3, 4}        # every layout for every head_dim
    assert {(c[1], c[4]) for c in cfgs} == {(hd, r) for hd in (64, 128) for r in (1, 2, 3, 4)}
    firsts = {}
    for c in cfgs:
        firsts.setdefault(c[1], c[4])
    assert firsts == {64: 4, 128: 4}                   # the defaults: fastest measured per head_dim
    for name, hd, stages, emu, layout, bm, bn in cfgs:
        assert f.smem_bytes(hd, stages, layout) <= 227 * 1024 and f.tmem_columns(hd) <= 512 and stages >= 3
        assert 0 <= emu <= 3 and name == f.config_name(hd, stages, emu, layout)
    assert not f.is_valid_config(128, 6, 1, 227 * 1024)   # 8 x 32 KiB tiles do not fit
    assert not f.is_valid_config(128, 5, 2, 227 * 1024)   # nor do 2 + 5 of them beside a staging box
    assert f.is_valid_config(128, 4, 2, 227 * 1024)
    assert not f.is_valid_config(256, 3, 1, 227 * 1024)
    # the environment inputs of the reference generator still work
    monkeypatch.setenv("FLASH_FWD_ONLY_CONFIGS", cfgs[0][0])
    monkeypatch.setenv("FLASH_FWD_MAX_SMEM_KB", "227")
    only = f.main(["--inc", str(tmp_path / "f.inc"), "--registry", str(tmp_path / "r.inc"),
                   "--output", str(tmp_path / "c.cmake")])
    assert [c[0] for c in only] == [cfgs[0][0]]
    assert "FLASH_FWD_DEFAULT_CONFIG" in (tmp_path / "c.cmake").read_text()


# --------------------------------------------------------------------- library surface
def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "b200dl.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 13
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(PKG, "libb200dl.so")],
                         capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r" T (b200_[a-z0-9_]+)", out))
    assert declared <= exported, f"declared but not exported: {sorted(declared - exported)}"
    from sm120_dl_b200 import capi
    assert set(capi.EXPORTS) <= exported


def test_config_tables_match_generators(lib):
    from sm120_dl_b200 import capi
    g = _import_from(os.path.join(PKG, "gemm"), "gemm_configs")
    f = _import_from(os.path.join(PKG, "flashattention"), "flash_configs")
    gc = capi.gemm_configs()
    assert [c["name"] for c in gc] == [c[0] for c in g.generate_configs(227) + g.generate_splitk_configs(227) +
                                       g.generate_tall_configs(227)]
    for c in gc:
        if c["bm"] == 512:
            assert c["smem_bytes"] == g.tall_smem_bytes(c["bn"], c["stages"])
            assert c["cta_group"] == 2 and c["acc_bufs"] == 2 and c["tmem_cols"] == 512 and c["bk"] == 64
            continue
        if c["split_k"] > 1:
            assert c["smem_bytes"] == g.splitk_smem_bytes(c["bn"], c["stages"])
            assert c["name"].endswith("_splitk%d" % c["split_k"]) and c["cta_group"] == 1
        else:
            assert c["smem_bytes"] == g.smem_bytes(c["bn"], c["stages"], c["cta_group"], c["acc_bufs"])
        assert c["tmem_cols"] == g.tmem_columns(c["bn"], c["acc_bufs"])
        assert c["bm"] == 128 * c["cta_group"] and c["bk"] == 64
    fc = capi.fa_configs()
    assert [c["name"] for c in fc] == [c[0] for c in f.generate_configs(227)]
    for c in fc:
        assert c["smem_bytes"] == f.smem_bytes(c["head_dim"], c["stages"], c["softmax_layout"])
        assert c["nwarps"] == f.NUM_WARPS[c["softmax_layout"]]


def test_config_lookup(lib):
    assert lib.b200_gemm_find_config(b"no_such_config") == -1
    assert lib.b200_gemm_find_config(None) == -1
    first = lib.b200_gemm_get_config(0).contents.name
    assert lib.b200_gemm_find_config(first) == 0
    assert not lib.b200_gemm_get_config(-1) and not lib.b200_gemm_get_config(10 ** 6)
    # 8192^3 gets the tall 512x256 CTA-pair tile, a shape whose last wave it would leave ragged
    # the 256x256 one; 512^3 a small tile that spreads over more SMs
    big = lib.b200_gemm_get_config(lib.b200_gemm_default_config(8192, 8192, 8192)).contents
    assert (big.bm, big.bn, big.cta_group, big.bs_w) == (512, 256, 2, 16)
    mid = lib.b200_gemm_get_config(lib.b200_gemm_default_config(16384, 1792, 4096)).contents
    assert (mid.bm, mid.bn, mid.cta_group) == (256, 256, 2)
    small = lib.b200_gemm_get_config(lib.b200_gemm_default_config(512, 512, 512)).contents
    assert small.bn == 64 and small.cta_group == 1
    ragged = lib.b200_gemm_get_config(lib.b200_gemm_default_config(100, 100, 100)).contents
    assert ragged.bm == 128 and ragged.bn == 64      # a ragged shape gets the tile that wastes least
    assert lib.b200_gemm_default_config(0, 100, 100) == -1
    for hd in (64, 128):
        idx = lib.b200_fa_default_config(hd)
        assert lib.b200_fa_get_config(idx).contents.head_dim == hd
    assert lib.b200_fa_default_config(96) == -1
    assert lib.b200_fa_find_config(b"nope") == -1
    assert b"b200dl" in lib.b200_version()


def test_argument_errors_need_no_gpu(lib):
    """Argument validation happens before any CUDA call, so it can be checked here."""
    assert lib.b200_gemm_bf16_tn(999, 256, 256, 64, 8, 64, 8, 64, 8, 256, None) == -1
    assert b"unknown GEMM config" in lib.b200_last_error()
    assert lib.b200_gemm_bf16_tn(0, 256, 256, 64, None, 64, None, 64, None, 256, None) == -1
    assert lib.b200_gemm_bf16_tn(0, 0, 256, 64, 8, 64, 8, 64, 8, 256, None) == -2
    assert b"must be positive" in lib.b200_last_error()
    assert lib.b200_gemm_bf16_tn(0, 256, 256, 64, 8, 60, 8, 64, 8, 256, None) == -1   # lda < K
    st = (ctypes.c_int64 * 3)(64 * 64, 64, 64)
    idx = lib.b200_fa_default_config(64)
    assert lib.b200_fa_fwd_fp16(idx, 8, 8, 8, 8, 1, 100, 100, 1, 64, st, st, st, st, 0.125, 0, None) == -2
    assert b"multiple of 64" in lib.b200_last_error()
    assert lib.b200_fa_fwd_fp16(idx, 8, 8, 8, 8, 1, 64, 64, 1, 128, st, st, st, st, 0.125, 0, None) == -2
    assert b"expects head_dim=64" in lib.b200_last_error()
    assert lib.b200_fa_fwd_fp16(idx, 8, 8, 8, 8, 1, 64, 128, 1, 64, st, st, st, st, 0.125, 1, None) == -2
    bad = (ctypes.c_int64 * 3)(64 * 64, 60, 64)
    assert lib.b200_fa_fwd_fp16(idx, 8, 8, 8, 8, 1, 64, 64, 1, 64, bad, st, st, st, 0.125, 0, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from sm120_dl_b200 import capi
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", str(tmp_path / "libb200dl.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        capi.lib()


# ----------------------------------------------------------------------------- sharding
def test_shard_bounds():
    from sm120_dl_b200.sharded import shard_bounds
    for total, world, gran in ((4096, 8, 256), (14336, 8, 256), (14336, 3, 256), (64, 8, 1), (5, 8, 1)):
        spans = [shard_bounds(total, world, r, gran) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((e - s) % gran == 0 for s, e in spans)
        sizes = [e - s for s, e in spans]
        assert max(sizes) - min(sizes) <= gran
    assert shard_bounds(14336, 8, 0, 256) == (0, 1792)
    with pytest.raises(ValueError):
        shard_bounds(100, 4, 0, 64)
    with pytest.raises(ValueError):
        shard_bounds(128, 4, 4, 1)


_GLOO_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from sm120_dl_b200 import sharded
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + os.environ["PORT"],
                        rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD"]))
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
a = torch.randn(64, 32); b = torch.randn(768, 32)            # 3 granules of 256: uneven over 2 ranks
def mm(x, y, out): out.copy_(x @ y.T)
full, (n0, n1) = sharded.gemm_column_shard(a, b, gather=True, granule=256, compute=mm)
assert torch.allclose(full, a @ b.T, atol=1e-5), "uneven gather"
slab, (n0, n1) = sharded.gemm_column_shard(a, b, gather=False, granule=256, compute=mm)
assert slab.shape == (64, n1 - n0) and torch.allclose(slab, (a @ b.T)[:, n0:n1], atol=1e-5)
b2 = torch.randn(512, 32)
full2, _ = sharded.gemm_column_shard(a, b2, gather=True, granule=256, compute=mm)
assert torch.allclose(full2, a @ b2.T, atol=1e-5), "even gather"
full3, _ = sharded.gemm_column_shard(a, b2, gather=True, granule=256, compute=mm, panels=4)
assert torch.equal(full3, full2), "row-panel pipelined gather"
full4, _ = sharded.gemm_column_shard(a, b, gather=True, granule=256, compute=mm, panels=4)   # uneven: plain path
assert torch.allclose(full4, a @ b.T, atol=1e-5), "uneven shards ignore panels"
q = torch.randn(2, 16, 6, 8); k = torch.randn(2, 16, 6, 8); v = torch.randn(2, 16, 6, 8)
def attn(x, y, z, causal):
    o = torch.nn.functional.scaled_dot_product_attention(x.permute(0, 2, 1, 3), y.permute(0, 2, 1, 3),
                                                         z.permute(0, 2, 1, 3), is_causal=causal)
    return o.permute(0, 2, 1, 3)
ref = attn(q, k, v, True)
o, (h0, h1) = sharded.attention_head_shard(q, k, v, causal=True, gather=True, compute=attn)
assert torch.allclose(o, ref, atol=1e-5), "head gather"
o5, _ = sharded.attention_head_shard(q[:, :, :5], k[:, :, :5], v[:, :, :5], causal=True, gather=True, compute=attn)
assert torch.allclose(o5, ref[:, :, :5], atol=1e-5), "uneven head gather"
part, (h0, h1) = sharded.attention_head_shard(q, k, v, causal=True, compute=attn)
assert (h0, h1) == sharded.shard_bounds(6, world, rank) and torch.allclose(part, ref[:, :, h0:h1], atol=1e-5)
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_gather_logic_two_ranks_gloo(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, REPO_ROOT=ROOT, PORT=str(port), RANK=str(rank), WORLD="2", OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for rank, p in enumerate(procs):
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0 and f"rank {rank} ok" in out, out[-2000:]


def test_extract_resources_maps_kernels_to_config_names(tmp_path):
    """The ptxas report parser names kernels like the registries do (reference tool:
    flashattention/v3_mMnNkN/extract_resources.py)."""
    import importlib.util
    path = os.path.join(ROOT, "sm120_dl_b200", "flashattention", "extract_resources.py")
    spec = importlib.util.spec_from_file_location("extract_resources", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    log = tmp_path / "build.log"
    log.write_text(
        "ptxas info    : Compiling entry function '_ZN4b2003_GLOBAL__N_13fa_fwd_kernelILi128ELi5ELi0EEEvPj' for 'sm_100a'\n"
        "ptxas info    : Function properties for x\n"
        "    8 bytes stack frame, 4 bytes spill stores, 12 bytes spill loads\n"
        "ptxas info    : Used 168 registers, used 16 barriers\n"
        "ptxas info    : Compiling entry function '_ZN4b20019gemm_bf16_tn_kernelILi256ELi6ELi2ELi2ELi1EEEvi' for 'sm_100a'\n"
        "    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads\n"
        "ptxas info    : Used 96 registers\n"
        "ptxas info    : Compiling entry function '_ZN4b20019gemm_bf16_tn_kernelILi256ELi4ELi2ELi2ELi2EEEvi' for 'sm_100a'\n"
        "    8 bytes stack frame, 4 bytes spill stores, 4 bytes spill loads\n"
        "ptxas info    : Used 168 registers\n"
        "ptxas info    : Compiling entry function '_ZN4b20016fa_fwd_ws_kernelILi64ELi8ELi1ELi1EEEvPj' for 'sm_100a'\n"
        "    40 bytes stack frame, 60 bytes spill stores, 88 bytes spill loads\n"
        "ptxas info    : Used 128 registers\n"
        "ptxas info    : Compiling entry function '_ZN4b20016fa_fwd_ws_kernelILi128ELi4ELi0ELi2EEEvPj' for 'sm_100a'\n"
        "    24 bytes stack frame, 40 bytes spill stores, 68 bytes spill loads\n"
        "ptxas info    : Used 80 registers\n")
    out = tmp_path / "resource.log"
    assert mod.main([str(log), str(out)]) == 0
    lines = out.read_text().splitlines()
    assert lines[0] == "func_name spill stack registers"
    assert lines[1] == "hd128_bm64_bn64_tq128x2_tk128_s5_e0_r1 16 8 168"
    assert lines[2] == "bf16_bm256_bn256_bk64_s6_cta2_acc2 0 0 96"
    assert lines[3] == "bf16_bm512_bn256_bk64_s4_cta2_acc2 8 8 168"
    assert lines[4] == "hd64_bm64_bn64_tq128x2_tk128_s8_e1_r3 148 40 128"
    assert lines[5] == "hd128_bm64_bn64_tq128x2_tk128_s4_e0_r2 108 24 80"
