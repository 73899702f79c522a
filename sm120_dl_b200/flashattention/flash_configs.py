#!/usr/bin/env python3
"""Enumerate the B200 (sm_100a) FlashAttention-forward configurations.

Plays the role of the reference generator flashattention/v3_*/flash_configs.py (config
enumeration and shared-memory model: flash_configs.py:41-62, 94-118; environment inputs
FLASH_FWD_OUTPUT / FLASH_FWD_MAX_SMEM_KB / FLASH_FWD_ONLY_CONFIGS: flash_configs.py:7-9),
with Blackwell's vocabulary instead of mma.sync warp grids:

  head_dim   64 or 128
  tile_q     128 query rows per MMA tile (= tensor-memory lanes), two tiles per CTA so the
             tensor core works on one tile while the other tile's softmax runs
  tile_kv    128 key/value rows per ring slot
  stages     ring slots shared by K and V blocks (K_0, V_0, K_1, V_1, ...)
  layout     how the softmax is laid over threads (the reference ships two warp layouts too,
             v3_mMnNkN and v3_mMn1k1):
               r2  two threads per query row (16 softmax warps), a correction warpgroup that
                   rescales O and writes the output, persistent CTAs; a 16 KiB staging box
                   for the output and 24 warps
               r3  the same warp-specialised persistent kernel with one softmax thread per
                   query row (8 softmax warps, 16 warps in all): no exchange of row maxima
                   between threads, 128 scores live per thread
               r4  r1 with persistent CTAs: barriers and tensor memory set up once per CTA, the
                   next unit's Q / K / V loads and first S issued under the current unit's
                   epilogue; a 16 KiB staging box per query tile for the output
               r1  one thread per query row (8 softmax warps) that also rescales O; one CTA
                   per 256 query rows, 12 warps
  emu        quarters of the exponentials evaluated by a polynomial on the FMA pipe
  block_m / block_n
             the sequence-length granularity the entry points accept (what the
             reference's harness checks with seq_len % block_m and % block_n); the kernel
             masks partial tiles, so this is 64 like the reference's default config

Budgets: 227 KiB shared memory; tensor memory 2 x 128 score columns + 2 x head_dim
output columns <= 512.  The first config listed for a head dimension is its default.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from genutil import write_if_changed  # noqa: E402

HEAD_DIMS = (64, 128)
TILE_Q = 128
Q_TILES = 2
TILE_KV = 128
SEQ_GRANULARITY = 64
LAYOUTS = (1, 2, 3, 4)
# order in which a head dimension's layouts are emitted; the first is its default (fastest
# measured, 50-launch runs: B4 H32 S4096 D128 r4 1231-1234 / r1 1205-1212 / r3 1050-1100 /
# r2 ~990 TFLOP/s; B16 H32 S2048 D64 r4 740 / r3 710 / r1 661-670 / r2 ~620)
LAYOUT_ORDER = {64: (4, 3, 1, 2), 128: (4, 1, 3, 2)}
STAGE_VALUES = {(64, 2): (8, 4), (128, 2): (4,), (64, 1): (8, 4), (128, 1): (5, 3), (64, 3): (8, 4), (128, 3): (4,),
                (64, 4): (10, 4), (128, 4): (4, 3)}
# Quarters of the exponentials evaluated by a polynomial on the FMA pipe instead of the SFU
# (the SFU's 16 ex2 per clock are the co-bottleneck at head_dim 128, the bottleneck at 64).
EMU_VALUES = {64: (1, 0, 2), 128: (0, 1, 2)}   # first = default (fastest measured)
NUM_WARPS = {2: 24, 1: 12, 3: 16, 4: 12}
DEFAULT_MAX_SMEM_KB = 227
SMEM_LIMIT = DEFAULT_MAX_SMEM_KB * 1024
TMEM_COLUMNS = 512


def tile_bytes(head_dim):
    return TILE_KV * head_dim * 2


def smem_bytes(head_dim, stages, layout):
    if layout == 4:
        # q_full, q_empty, ring full/empty, s_full[2], p_full[2][2], o_final[2]; one 128 x 64
        # staging box per query tile
        barriers = (2 + 2 * stages + 2 + 4 + 2) * 8 + 16
        return (Q_TILES + stages) * tile_bytes(head_dim) + Q_TILES * 128 * 128 + barriers + 1024
    if layout >= 2:
        # q_full, q_empty, ring full/empty, s_full[2], p_full[2][2], max_full[2][4],
        # o_final[2], sum_full[2], sum_empty[2]; row maxima [2][2][2][128] and row sums
        # [2][2][128] in fp32 (sized for two threads per row); one 128 x 64 staging box for the output
        barriers = (2 + 2 * stages + 2 + 4 + 8 + 2 + 2 + 2) * 8 + 16
        small = 2 * 2 * 2 * TILE_Q * 4 + 2 * 2 * TILE_Q * 4 + barriers
        return (Q_TILES + stages) * tile_bytes(head_dim) + 128 * 128 + small + 1024
    barriers = (1 + 2 * stages + 2 + 4) * 8 + 16   # q_full, ring full/empty, s_full[2], p_full[2][2]
    return (Q_TILES + stages) * tile_bytes(head_dim) + barriers + 1024


def tmem_columns(head_dim):
    return Q_TILES * TILE_KV + Q_TILES * head_dim


def config_name(head_dim, stages, emu, layout):
    return (f"hd{head_dim}_bm{SEQ_GRANULARITY}_bn{SEQ_GRANULARITY}_tq{TILE_Q}x{Q_TILES}_tk{TILE_KV}"
            f"_s{stages}_e{emu}_r{layout}")


def is_valid_config(head_dim, stages, layout, max_smem):
    if head_dim not in HEAD_DIMS or stages < 3:   # V_j and K_{j+1} are live together, +1 to prefetch
        return False
    if layout not in LAYOUTS:
        return False
    if tmem_columns(head_dim) > TMEM_COLUMNS:
        return False
    return smem_bytes(head_dim, stages, layout) <= max_smem


def generate_configs(max_smem_kb, only=None):
    max_smem = max_smem_kb * 1024
    configs = []
    for head_dim in HEAD_DIMS:
        for layout in LAYOUT_ORDER[head_dim]:
            stage_values = STAGE_VALUES[(head_dim, layout)]
            for stages in stage_values:
                if not is_valid_config(head_dim, stages, layout, max_smem):
                    continue
                # every polynomial share for the deepest ring, the first share only for the others
                emus = EMU_VALUES[head_dim] if stages == stage_values[0] else EMU_VALUES[head_dim][:1]
                for emu in emus:
                    name = config_name(head_dim, stages, emu, layout)
                    if only and name not in only:
                        continue
                    configs.append((name, head_dim, stages, emu, layout, SEQ_GRANULARITY, SEQ_GRANULARITY))
    return configs


def write_inc(path, configs, max_smem_kb):
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with write_if_changed(path) as f:
        f.write("// Auto-generated by flash_configs.py - do not edit\n")
        f.write(f"// {len(configs)} configs, max dynamic shared memory {max_smem_kb} KiB\n")
        f.write("// B200_FA_CONFIG(name, HEAD_DIM, STAGES, EMU, LAYOUT, BLOCK_M, BLOCK_N)\n")
        for name, head_dim, stages, emu, layout, bm, bn in configs:
            f.write(f'B200_FA_CONFIG("{name}", {head_dim}, {stages}, {emu}, {layout}, {bm}, {bn})\n')


def write_registry(path, configs):
    """Entries of kFlashFwdConfigs[] for pybind/flash_fwd_config_registry.cpp, in the same
    order as the table inside libb200dl.so."""
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with write_if_changed(path) as f:
        f.write("// Auto-generated by flash_configs.py - do not edit\n")
        f.write("// B200_FA_ENTRY(index, name, HEAD_DIM, BLOCK_M, BLOCK_N, NWARPS, STAGES)\n")
        for i, (name, head_dim, stages, emu, layout, bm, bn) in enumerate(configs):
            f.write(f'B200_FA_ENTRY({i}, "{name}", {head_dim}, {bm}, {bn}, {NUM_WARPS[layout]}, {stages})\n')


def write_cmake(path, configs, max_smem_kb):
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with write_if_changed(path) as f:
        f.write("# Auto-generated by flash_configs.py - do not edit\n")
        f.write(f"set(FLASH_FWD_MAX_SMEM_BYTES {max_smem_kb * 1024})\n")
        f.write("set(FLASH_FWD_CONFIGS\n")
        for name, head_dim, stages, emu, layout, bm, bn in configs:
            # head_dim|block_m|block_n|tile_q|q_tiles|tile_kv|nwarps|stage|smem_bytes|name
            row = (head_dim, bm, bn, TILE_Q, Q_TILES, TILE_KV, NUM_WARPS[layout], stages,
                   smem_bytes(head_dim, stages, layout), name)
            f.write('    "' + "|".join(str(x) for x in row) + '"\n')
        f.write(")\n")
        f.write(f'set(FLASH_FWD_DEFAULT_CONFIG "{configs[0][0]}")\n')


def main(argv=None):
    here = os.path.dirname(os.path.abspath(__file__))
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--output", default=os.environ.get("FLASH_FWD_OUTPUT"),
                        help="configs.cmake path (reference-compatible variables)")
    parser.add_argument("--inc", default=os.path.join(here, "..", "csrc", "generated", "flash_configs.inc"))
    parser.add_argument("--registry",
                        default=os.path.join(here, "pybind", "generated", "flash_registry_entries.inc"))
    parser.add_argument("--max-smem-kb", type=int,
                        default=int(os.environ.get("FLASH_FWD_MAX_SMEM_KB", DEFAULT_MAX_SMEM_KB)))
    args = parser.parse_args(argv)
    only = [c for c in os.environ.get("FLASH_FWD_ONLY_CONFIGS", "").replace(";", ",").split(",") if c]
    configs = generate_configs(args.max_smem_kb, only or None)
    if not configs:
        raise RuntimeError("no valid flash_fwd configs generated")
    write_inc(args.inc, configs, args.max_smem_kb)
    write_registry(args.registry, configs)
    if args.output:
        write_cmake(args.output, configs, args.max_smem_kb)
    print(f"Generated {len(configs)} configs -> {os.path.normpath(args.inc)}")
    return configs


if __name__ == "__main__":
    main()
