"""In-tree build of the native pieces with nvcc / g++ (no CMake needed).

  libb200dl.so            csrc/*.cu  -> the C ABI library (sm_100a only)
  gemm/test_gemm_cute     the reference-compatible GEMM harness (C++), links libb200dl.so
  gemm/test_gemm_multi_gpu  the N-column-sharded GEMM over the GPUs of one box (C++, one thread
                          per device, NCCL for the baseline gather)
  flashatten_v3_sm120.so  the pybind/torch extension mirroring the reference's module

Run as `python -m sm120_dl_b200.build [targets...]`; with no targets everything is built.
Outputs are git-ignored; they are rebuilt whenever a source is newer than the output.
"""

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200dl.so")
GEMM_DIR = os.path.join(HERE, "gemm")
FA_DIR = os.path.join(HERE, "flashattention")

NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
HOST_CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-ccbin", HOST_CXX] + ARCH_FLAGS


def _newer(srcs, out):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs if os.path.exists(s))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"build step failed: {' '.join(cmd)}")
    return proc.stdout


def generate_configs(verbose=False):
    """Run the two config generators (they write csrc/generated/*.inc)."""
    sys.path.insert(0, GEMM_DIR)
    sys.path.insert(0, FA_DIR)
    try:
        import contextlib
        import io
        import gemm_configs
        import flash_configs
        with contextlib.redirect_stdout(io.StringIO()):
            gemm_configs.main([])
            flash_configs.main([])
    finally:
        sys.path.remove(GEMM_DIR)
        sys.path.remove(FA_DIR)


def build_lib(force=False, verbose=False, ptxas_verbose=False):
    gen_dir = os.path.join(CSRC, "generated")
    generators = [os.path.join(GEMM_DIR, "gemm_configs.py"), os.path.join(FA_DIR, "flash_configs.py")]
    incs = [os.path.join(gen_dir, "gemm_configs.inc"), os.path.join(gen_dir, "flash_configs.inc")]
    generate_configs(verbose)  # cheap; files are rewritten only when their content changes
    units = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers += [os.path.join(ROOT, "include", "b200dl.h")] + [i for i in incs if os.path.exists(i)]
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for u in units:
        src = os.path.join(CSRC, u)
        obj = os.path.join(HERE, "build", u[:-3] + ".o")
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            cmd = [NVCC] + NVCC_FLAGS + ["-Xcompiler", "-fPIC", "-c", src, "-o", obj]
            if ptxas_verbose:
                cmd += ["-Xptxas", "-v"]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    report = []
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"build step failed: {' '.join(cmd)}")
        if ptxas_verbose:
            print(out)
            report.append(out)
    if ptxas_verbose and report:
        # input of flashattention/extract_resources.py
        with open(os.path.join(HERE, "build", "build.log"), "w") as f:
            f.write("\n".join(report))
    if force or procs or _newer(objs, LIB):
        tmp = LIB + ".tmp"
        _run([NVCC] + ARCH_FLAGS + ["-ccbin", HOST_CXX, "-shared", "-o", tmp] + objs + ["-lcudart"], verbose)
        os.replace(tmp, LIB)
    return LIB


def build_test_gemm_cute(force=False, verbose=False):
    src = os.path.join(GEMM_DIR, "test.cpp")
    out = os.path.join(GEMM_DIR, "test_gemm_cute")
    if not os.path.exists(src):
        return None
    deps = [src, os.path.join(GEMM_DIR, "gemm_config_registry.hpp"), os.path.join(GEMM_DIR, "gemm_config_registry.cpp"),
            os.path.join(ROOT, "include", "b200dl.h"), LIB]
    if force or _newer(deps, out):
        tmp = out + ".tmp"
        _run([NVCC] + NVCC_FLAGS + ["-x", "cu", src, os.path.join(GEMM_DIR, "gemm_config_registry.cpp"),
              "-I", os.path.join(ROOT, "include"), "-I", GEMM_DIR, "-o", tmp, "-L", HERE, "-lb200dl",
              "-lcublas", "-Xcompiler", "-fopenmp", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."], verbose)
        os.replace(tmp, out)
    return out


def build_test_gemm_multi_gpu(force=False, verbose=False):
    src = os.path.join(GEMM_DIR, "multi_gpu_gemm.cpp")
    out = os.path.join(GEMM_DIR, "test_gemm_multi_gpu")
    if not os.path.exists(src):
        return None
    deps = [src, os.path.join(ROOT, "include", "b200dl.h"), LIB]
    if force or _newer(deps, out):
        tmp = out + ".tmp"
        _run([NVCC] + NVCC_FLAGS + ["-x", "cu", src, "-I", os.path.join(ROOT, "include"), "-o", tmp, "-L", HERE,
              "-lb200dl", "-lcublas", "-lnccl", "-Xcompiler", "-pthread", "-Xlinker", "-rpath", "-Xlinker",
              "$ORIGIN/.."], verbose)
        os.replace(tmp, out)
    return out


def build_fa_module(force=False, verbose=False):
    src = os.path.join(FA_DIR, "pybind", "flashatten_v3_pybind.cpp")
    if not os.path.exists(src):
        return None
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = os.path.join(FA_DIR, "pybind", "build", "flashatten_v3_sm120" + suffix)
    os.makedirs(os.path.dirname(out), exist_ok=True)
    deps = [src, os.path.join(FA_DIR, "pybind", "flash_fwd_config_registry.hpp"),
            os.path.join(FA_DIR, "pybind", "flash_fwd_config_registry.cpp"),
            os.path.join(ROOT, "include", "b200dl.h"), LIB]
    if force or _newer(deps, out):
        import torch
        from torch.utils import cpp_extension
        inc = []
        for p in cpp_extension.include_paths():
            inc += ["-I", p]
        inc += ["-I", sysconfig.get_paths()["include"], "-I", os.path.join(ROOT, "include"),
                "-I", os.path.join(FA_DIR, "pybind"), "-I", "/usr/local/cuda/include"]
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        tmp = out + ".tmp"
        cmd = [HOST_CXX, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-DTORCH_EXTENSION_NAME=flashatten_v3_sm120", "-DTORCH_API_INCLUDE_EXTENSION_H",
               src, os.path.join(FA_DIR, "pybind", "flash_fwd_config_registry.cpp")] + inc + [
               "-o", tmp, "-L", torch_lib, "-L", HERE, "-L", "/usr/local/cuda/lib64",
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
               "-lb200dl", f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN/../../.."]
        _run(cmd, verbose)
        os.replace(tmp, out)
    return out


def build_all(force=False, verbose=False):
    outs = {"lib": build_lib(force, verbose)}
    outs["test_gemm_cute"] = build_test_gemm_cute(force, verbose)
    outs["test_gemm_multi_gpu"] = build_test_gemm_multi_gpu(force, verbose)
    outs["fa_module"] = build_fa_module(force, verbose)
    return outs


if __name__ == "__main__":
    args = sys.argv[1:]
    force = "--force" in args
    verbose = "-v" in args or "--verbose" in args
    ptxas = "--ptxas" in args
    targets = [a for a in args if not a.startswith("-")] or ["all"]
    for t in targets:
        if t == "all":
            print(build_all(force, verbose))
        elif t == "lib":
            print(build_lib(force, verbose, ptxas))
        elif t == "test_gemm_cute":
            build_lib(False, verbose)
            print(build_test_gemm_cute(force, verbose))
        elif t == "test_gemm_multi_gpu":
            build_lib(False, verbose)
            print(build_test_gemm_multi_gpu(force, verbose))
        elif t == "fa_module":
            build_lib(False, verbose)
            print(build_fa_module(force, verbose))
        else:
            raise SystemExit(f"unknown target {t}")
