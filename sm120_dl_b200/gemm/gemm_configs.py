#!/usr/bin/env python3
"""Enumerate the B200 (sm_100a) GEMM configurations and write the registry inputs.

Plays the role of the reference generator gemm/gemm_configs.py (generate_configs,
is_valid_config, smem_bytes, config_name, main: gemm/gemm_configs.py:28-158), but the
vocabulary is Blackwell's: instead of warp grids for mma.sync it chooses

  cta_group   1 = single-CTA tcgen05.mma (128 x BN x 16), 2 = CTA-pair MMA (256 x BN x 16,
              cluster of two CTAs along M, each CTA stages half of the B tile)
  bn          N extent of one MMA instruction = output tile width (64..256)
  stages      depth of the TMA -> MMA shared-memory ring (k-blocks of 64 elements)
  acc_bufs    tensor-memory accumulator buffers; 2 lets the epilogue of tile i overlap the
              mainloop of tile i+1
  bs_w        raster strip width in N-tiles (same idea as block_swizzle<BS_W>,
              utils/tools.h:30-40)
  split_k     split-K configs (for shapes with too few tiles to occupy the GPU, e.g. M = 128
              with a long K): a cluster of split_k CTAs shares one 128 x bn tile, each CTA
              accumulates its share of K and the partial tiles are summed through
              distributed shared memory

  tall tiles  512 x bn tiles of a CTA pair: each CTA works on two 128-row halves of A against
              the same B block, one accumulator per half (all 512 tensor-memory columns), so a B
              block fetched from L2 feeds twice the arithmetic: a quarter fewer operand bytes
              per flop than the 256 x 256 pair tile, at the price of an epilogue that overlaps
              the next mainloop by one accumulator instead of a whole tile

Legality is decided by the hardware budgets of one SM: 227 KiB of shared memory, 512
tensor-memory columns, tcgen05.mma shape rules.  Two files are written: a C include with
one B200_GEMM_CONFIG(...) line per config (compiled into libb200dl.so) and, for drop-in
compatibility with the reference's CMake flow, a configs.cmake with the same
GEMM_TN_MAX_SMEM_BYTES / GEMM_TN_CONFIGS / GEMM_TN_DEFAULT_CONFIG variables.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from genutil import write_if_changed  # noqa: E402

ELEMENT_BYTES = 2
BK = 64                       # one 128-byte swizzle row of bf16
CTA_M = 128                   # accumulator rows per CTA = tensor-memory lanes
TMEM_COLUMNS = 512
EPILOGUE_BYTES = 4 * 2 * 32 * 128   # 4 warps x 2 boxes x (32 rows x 128 B)
ALIGN_SLACK = 1024            # the ring must start on a 1024-byte boundary
DEFAULT_MAX_SMEM_KB = 227

CTA_GROUP_VALUES = (2, 1)
BN_VALUES = (256, 192, 128, 64)
STAGE_VALUES = (3, 4, 5, 6, 8)
ACC_BUF_VALUES = (1, 2)
BS_W_VALUES = (4, 8, 16)

DEFAULT_NAME = "bf16_bm256_bn256_bk64_s6_cta2_acc2_bsw8"


def stage_bytes(bn, cta_group):
    """Bytes one CTA stages per k-block: its 128 rows of A plus its share of B."""
    return (CTA_M * BK + (bn // cta_group) * BK) * ELEMENT_BYTES


def smem_bytes(bn, stages, cta_group, acc_bufs):
    barrier_bytes = (2 * stages + 2 * acc_bufs) * 8 + 16
    return stages * stage_bytes(bn, cta_group) + EPILOGUE_BYTES + barrier_bytes + ALIGN_SLACK


def tmem_columns(bn, acc_bufs):
    need = bn * acc_bufs
    cols = 32
    while cols < need:
        cols *= 2
    return cols


def config_name(bn, stages, cta_group, acc_bufs, bs_w):
    return (f"bf16_bm{CTA_M * cta_group}_bn{bn}_bk{BK}_s{stages}"
            f"_cta{cta_group}_acc{acc_bufs}_bsw{bs_w}")


def is_valid_config(bn, stages, cta_group, acc_bufs, bs_w, max_smem):
    if cta_group not in (1, 2) or stages < 2 or acc_bufs < 1 or bs_w < 1:
        return False
    # tcgen05.mma kind::f16 with M = 128 per CTA: N multiple of 16, 16..256.
    if bn % 16 != 0 or bn < 16 or bn > 256:
        return False
    # The epilogue stores 64-column boxes; B rows per CTA must fill whole 8-row swizzle groups.
    if bn % 64 != 0 or (bn // cta_group) % 8 != 0:
        return False
    if bn * acc_bufs > TMEM_COLUMNS:
        return False
    if smem_bytes(bn, stages, cta_group, acc_bufs) > max_smem:
        return False
    return True


def generate_configs(max_smem_kb, full=False):
    """Returns a list of (name, bn, stages, cta_group, acc_bufs, bs_w).

    The default list keeps, per (cta_group, bn), the deepest ring that fits plus one
    shallower ring, with double-buffered accumulators where they fit; `full` keeps
    every legal combination (used to sweep on the GPU).
    """
    max_smem = max_smem_kb * 1024
    configs = []
    for cta_group in CTA_GROUP_VALUES:
        for bn in BN_VALUES:
            legal_stages = [s for s in STAGE_VALUES
                            if is_valid_config(bn, s, cta_group, 1, 8, max_smem)]
            if not legal_stages:
                continue
            stage_pick = legal_stages if full else sorted(set(legal_stages[-2:]))
            for stages in stage_pick:
                acc_pick = [a for a in ACC_BUF_VALUES
                            if is_valid_config(bn, stages, cta_group, a, 8, max_smem)]
                if not full:
                    acc_pick = acc_pick[-1:]
                for acc_bufs in acc_pick:
                    widths = BS_W_VALUES if (full or bn == 256) else (8,)
                    for bs_w in widths:
                        if not is_valid_config(bn, stages, cta_group, acc_bufs, bs_w, max_smem):
                            continue
                        configs.append((config_name(bn, stages, cta_group, acc_bufs, bs_w),
                                        bn, stages, cta_group, acc_bufs, bs_w))
    return configs


SPLITK_BN_VALUES = (64, 128, 256)
SPLITK_VALUES = (2, 4, 8)          # cluster sizes; 8 is the portable maximum


def splitk_smem_bytes(bn, stages):
    barrier_bytes = (2 * stages + 1) * 8 + 16
    return stages * stage_bytes(bn, 1) + barrier_bytes + ALIGN_SLACK


def splitk_config_name(bn, stages, split_k):
    return f"bf16_bm{CTA_M}_bn{bn}_bk{BK}_s{stages}_cta1_splitk{split_k}"


def generate_splitk_configs(max_smem_kb):
    """Returns a list of (name, bn, stages, split_k): per tile width the deepest ring that
    fits (the fp32 partial tile, 128 x bn x 4 bytes, reuses the drained ring)."""
    max_smem = max_smem_kb * 1024
    configs = []
    for bn in SPLITK_BN_VALUES:
        legal = [s for s in STAGE_VALUES
                 if splitk_smem_bytes(bn, s) <= max_smem and s * stage_bytes(bn, 1) >= CTA_M * bn * 4]
        if not legal:
            continue
        stages = legal[-1]
        for split_k in SPLITK_VALUES:
            configs.append((splitk_config_name(bn, stages, split_k), bn, stages, split_k))
    return configs


TALL_BN_VALUES = (256,)
TALL_STAGE_VALUES = (3, 4)
# a wave of 74 tile pairs is closest to square (fewest distinct A and B rows) at 12 tiles x 6
TALL_BS_W_VALUES = (8, 12, 16)


def tall_smem_bytes(bn, stages):
    barrier_bytes = (2 * stages + 4) * 8 + 16
    stage = (2 * CTA_M * BK + (bn // 2) * BK) * ELEMENT_BYTES
    return stages * stage + EPILOGUE_BYTES + barrier_bytes + ALIGN_SLACK


def tall_config_name(bn, stages, bs_w):
    return f"bf16_bm{4 * CTA_M}_bn{bn}_bk{BK}_s{stages}_cta2_acc2_bsw{bs_w}"


def generate_tall_configs(max_smem_kb):
    """Returns a list of (name, bn, stages, bs_w): CTA-pair configs with two accumulators per
    CTA (512-row tiles), every ring depth that fits, every strip width."""
    max_smem = max_smem_kb * 1024
    configs = []
    for bn in TALL_BN_VALUES:
        if 2 * bn > TMEM_COLUMNS:
            continue
        for stages in TALL_STAGE_VALUES:
            if tall_smem_bytes(bn, stages) > max_smem:
                continue
            for bs_w in TALL_BS_W_VALUES:
                configs.append((tall_config_name(bn, stages, bs_w), bn, stages, bs_w))
    return configs


def write_inc(path, configs, max_smem_kb, splitk=(), tall=()):
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with write_if_changed(path) as f:
        f.write("// Auto-generated by gemm_configs.py - do not edit\n")
        f.write(f"// {len(configs) + len(splitk) + len(tall)} configs, max dynamic shared memory {max_smem_kb} KiB\n")
        f.write("// B200_GEMM_CONFIG(name, BN, STAGES, CTA_GROUP, ACC_BUFS, BS_W)\n")
        for name, bn, stages, cta_group, acc_bufs, bs_w in configs:
            f.write(f'B200_GEMM_CONFIG("{name}", {bn}, {stages}, {cta_group}, {acc_bufs}, {bs_w})\n')
        f.write("// B200_GEMM_SPLITK_CONFIG(name, BN, STAGES, SPLIT_K)\n")
        for name, bn, stages, split_k in splitk:
            f.write(f'B200_GEMM_SPLITK_CONFIG("{name}", {bn}, {stages}, {split_k})\n')
        f.write("// B200_GEMM_TALL_CONFIG(name, BN, STAGES, BS_W)\n")
        for name, bn, stages, bs_w in tall:
            f.write(f'B200_GEMM_TALL_CONFIG("{name}", {bn}, {stages}, {bs_w})\n')


def write_registry(path, configs, splitk=(), tall=()):
    """Entries of kGemmConfigs[] for gemm_config_registry.cpp: one line per config, the
    index being the config's position in libb200dl.so's own table."""
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with write_if_changed(path) as f:
        f.write("// Auto-generated by gemm_configs.py - do not edit\n")
        f.write("// B200_GEMM_ENTRY(index, name, BM, BN, BK, STAGES, CTA_GROUP, ACC_BUFS, BS_W)\n")
        for i, (name, bn, stages, cta_group, acc_bufs, bs_w) in enumerate(configs):
            f.write(f'B200_GEMM_ENTRY({i}, "{name}", {CTA_M * cta_group}, {bn}, {BK}, {stages}, '
                    f'{cta_group}, {acc_bufs}, {bs_w})\n')
        for i, (name, bn, stages, split_k) in enumerate(splitk, start=len(configs)):
            # bk = 64 * split_k: "K divisible by bk" is how the harness decides run vs skipped,
            # and a split-K config needs at least one k-block per CTA of its cluster
            f.write(f'B200_GEMM_ENTRY({i}, "{name}", {CTA_M}, {bn}, {BK * split_k}, {stages}, 1, 1, 1)\n')
        for i, (name, bn, stages, bs_w) in enumerate(tall, start=len(configs) + len(splitk)):
            f.write(f'B200_GEMM_ENTRY({i}, "{name}", {4 * CTA_M}, {bn}, {BK}, {stages}, 2, 2, {bs_w})\n')


def write_cmake(path, configs, max_smem_kb):
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    default = next((c for c in configs if c[0] == DEFAULT_NAME), configs[0])

    def row(c):
        name, bn, stages, cta_group, acc_bufs, bs_w = c
        # type|type_cpp|BM|BN|BK|STAGE|CTA_GROUP|ACC_BUFS|BS_W|name
        return "|".join(str(x) for x in ("bf16", "bf16", CTA_M * cta_group, bn, BK, stages,
                                         cta_group, acc_bufs, bs_w, name))

    with write_if_changed(path) as f:
        f.write("# Auto-generated by gemm_configs.py - do not edit\n")
        f.write(f"# {len(configs)} configs, max dynamic shared memory {max_smem_kb} KiB\n\n")
        f.write(f"set(GEMM_TN_MAX_SMEM_BYTES {max_smem_kb * 1024})\n")
        f.write("set(GEMM_TN_CONFIGS\n")
        for c in configs:
            f.write(f'    "{row(c)}"\n')
        f.write(")\n")
        f.write(f'set(GEMM_TN_DEFAULT_CONFIG "{row(default)}")\n')


def main(argv=None):
    here = os.path.dirname(os.path.abspath(__file__))
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--output", default=None,
                        help="configs.cmake path (reference-compatible variables)")
    parser.add_argument("--inc", default=os.path.join(here, "..", "csrc", "generated", "gemm_configs.inc"),
                        help="C include consumed by csrc/gemm_sm100.cu")
    parser.add_argument("--registry", default=os.path.join(here, "generated", "gemm_registry_entries.inc"),
                        help="table entries consumed by gemm_config_registry.cpp")
    parser.add_argument("--max-smem-kb", type=int, default=DEFAULT_MAX_SMEM_KB)
    parser.add_argument("--full", action="store_true", help="emit every legal combination")
    args = parser.parse_args(argv)

    configs = generate_configs(args.max_smem_kb, full=args.full)
    if not configs:
        raise RuntimeError("no valid GEMM configs generated")
    splitk = generate_splitk_configs(args.max_smem_kb)
    tall = generate_tall_configs(args.max_smem_kb)
    write_inc(args.inc, configs, args.max_smem_kb, splitk, tall)
    write_registry(args.registry, configs, splitk, tall)
    if args.output:
        write_cmake(args.output, configs, args.max_smem_kb)
    print(f"Generated {len(configs)} + {len(splitk)} split-K + {len(tall)} tall configs -> {os.path.normpath(args.inc)}")
    return configs


if __name__ == "__main__":
    main()
