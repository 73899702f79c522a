#!/usr/bin/env python3
"""Turn the ptxas report of a library build into a per-kernel resource table.

Same job and output format as the reference tool
(flashattention/v3_mMnNkN/extract_resources.py:8-76: reads the build log, writes
`resource.log` with one `func_name spill stack registers` row per kernel), for the kernels
of libb200dl.so.  The log is what `python -m sm120_dl_b200.build lib --force --ptxas`
prints (and stores as sm120_dl_b200/build/build.log).  Mangled kernel names are mapped back
to config names:

    fa_fwd_ws_kernel<D, STAGES, EMU, TPR>             -> hd{D}_..._s{STAGES}_e{EMU}_r2 (TPR 2) or _r3 (TPR 1)
    fa_fwd_kernel<D, STAGES, EMU>                     -> hd{D}_..._s{STAGES}_e{EMU}_r1
    gemm_bf16_tn_kernel<BN, STAGES, CTA_GROUP, ACC, MH> -> bf16_bm{128*CTA_GROUP*MH}_bn{BN}_bk64_s{STAGES}_cta{..}_acc{..}
                                                         (the raster width is a launch argument)

    python extract_resources.py [build.log] [resource.log]
"""

import argparse
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(HERE)
DEFAULT_INPUT = os.path.join(PACKAGE, "build", "build.log")
DEFAULT_OUTPUT = os.path.join(PACKAGE, "build", "resource.log")

ENTRY = re.compile(r"Compiling entry function '([^']+)'")
FRAME = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
USED = re.compile(r"Used (\d+) registers")
FA_ARGS = re.compile(r"fa_fwd(_ws)?_kernelILi(\d+)ELi(\d+)ELi(\d+)E(?:Li(\d+)E)?E")
GEMM_ARGS = re.compile(r"gemm_bf16_tn_kernelILi(\d+)ELi(\d+)ELi(\d+)ELi(\d+)ELi(\d+)EE")


def kernel_label(mangled):
    m = FA_ARGS.search(mangled)
    if m:
        sys.path.insert(0, HERE)
        try:
            import flash_configs
        finally:
            sys.path.remove(HERE)
        head_dim, stages, emu = (int(x) for x in m.groups()[1:4])
        layout = 1 if not m.group(1) else (3 if m.group(5) == "1" else 2)
        return flash_configs.config_name(head_dim, stages, emu, layout)
    m = GEMM_ARGS.search(mangled)
    if m:
        bn, stages, cta_group, acc, halves = (int(x) for x in m.groups())
        return f"bf16_bm{128 * cta_group * halves}_bn{bn}_bk64_s{stages}_cta{cta_group}_acc{acc}"
    return mangled


def parse(text):
    """Rows (label, spill bytes, stack bytes, registers) in log order."""
    rows = []
    label = frame = None
    for line in text.splitlines():
        m = ENTRY.search(line)
        if m:
            label, frame = kernel_label(m.group(1)), None
            continue
        if label is None:
            continue
        m = FRAME.search(line)
        if m:
            frame = (int(m.group(2)) + int(m.group(3)), int(m.group(1)))
            continue
        m = USED.search(line)
        if m and frame is not None:
            rows.append((label, frame[0], frame[1], int(m.group(1))))
            label = frame = None
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("input", nargs="?", default=DEFAULT_INPUT)
    ap.add_argument("output", nargs="?", default=DEFAULT_OUTPUT)
    args = ap.parse_args(argv)
    with open(args.input, errors="replace") as f:
        rows = parse(f.read())
    os.makedirs(os.path.dirname(os.path.abspath(args.output)), exist_ok=True)
    with open(args.output, "w") as f:
        f.write("func_name spill stack registers\n")
        for row in rows:
            f.write("%s %d %d %d\n" % row)
    print(f"{len(rows)} kernels -> {args.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
