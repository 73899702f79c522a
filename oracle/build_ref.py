#!/usr/bin/env python3
"""Build oracle/_ref/libsm120ref.so: the reference project's own GEMM and attention kernels,
compiled for sm_100a from its sources where they lie.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [--reference DIR] [--force]

DIR is a checkout of HugeOrca/sm120-dl (default: the environment variable
SM120_DL_REFERENCE_DIR, else a directory named `reference` beside this repository).  The
reference's CMake files target sm_120a and a conda layout, so they are not used: the few
translation units are compiled directly with nvcc.  Its CUTLASS/CuTe submodule is not
vendored; the headers are taken from a CUTLASS tree installed with a Python package on this
image (flashinfer's data/cutlass, else tilelang's 3rdparty/cutlass).

Outputs go to oracle/_ref/ only (git-ignored).  The library is a same-box witness: the
parity tests feed it and the product kernels the same inputs and hold both to the CPU
oracle; oracle/ref_witness.py times it for the comparison tables.  Nothing in the product or in the
benchmark's timed region loads it.
"""

import argparse
import importlib.util
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libsm120ref.so")
WRAPPER = os.path.join(HERE, "ref_kernels.cu")

# (head_dim, head_num) pairs of flash_fwd instantiated; the head count is a template
# parameter in the reference (pybind/flash_fwd_config.cu.in:66-90 lists 1,4,8,16,32,64,80).
FA_UNITS = [(128, 4), (128, 32), (64, 4), (64, 32)]


def reference_dir(explicit=None):
    cand = explicit or os.environ.get("SM120_DL_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    if os.path.isfile(os.path.join(cand, "gemm", "gemm_cute.hpp")):
        return cand
    return None


def cutlass_include_dirs():
    for pkg, rel in (("flashinfer", os.path.join("data", "cutlass")), ("tilelang", os.path.join("3rdparty", "cutlass"))):
        spec = importlib.util.find_spec(pkg)
        if spec is None or not spec.submodule_search_locations:
            continue
        base = os.path.join(list(spec.submodule_search_locations)[0], rel)
        if os.path.isfile(os.path.join(base, "include", "cute", "tensor.hpp")):
            return [os.path.join(base, "include"), os.path.join(base, "tools", "util", "include")]
    return None


def build(reference=None, force=False, quiet=False):
    ref = reference_dir(reference)
    if ref is None:
        raise RuntimeError("reference checkout not found (pass --reference or set SM120_DL_REFERENCE_DIR)")
    cutlass = cutlass_include_dirs()
    if cutlass is None:
        raise RuntimeError("no CUTLASS/CuTe header tree found on this image")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(WRAPPER):
        return LIB
    common = [nvcc, "-std=c++20", "-O3", "--expt-relaxed-constexpr", "--expt-extended-lambda",
              "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-w",
              "-I", ref, "-I", cutlass[0], "-I", cutlass[1]]
    units = [("gemm", ["-DREF_UNIT_GEMM", "-I", os.path.join(ref, "gemm")])]
    for d, h in FA_UNITS:
        units.append((f"fa_d{d}_h{h}", ["-DREF_UNIT_FA", f"-DREF_FA_D={d}", f"-DREF_FA_H={h}",
                                        "-I", os.path.join(ref, "flashattention", "v3_mMnNkN")]))
    procs, objs = [], []
    for name, flags in units:
        obj = os.path.join(OUT_DIR, name + ".o")
        objs.append(obj)
        cmd = common + flags + ["-c", WRAPPER, "-o", obj]
        procs.append((name, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for name, cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(out[-4000:])
            raise RuntimeError(f"reference unit {name} failed to compile: {' '.join(cmd)}")
        if not quiet:
            print(f"compiled {name}")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lcudart"],
                   check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
