// BF16 GEMM  C[M,N] = A[M,K] * B[N,K]^T  for sm_100a, and its C ABI.
//
// Same contract as the reference's gemm_tn / b16_gemm (gemm/gemm_cute.hpp:64-356): both
// operands K-major ("TN"), fp32 accumulation, bf16 round-to-nearest-even output, C fully
// overwritten, persistent CTAs walking a strip-rasterised tile list
// (utils/tools.h:30-40).  Everything below that contract is new:
//
//   warp 0  (1 thread)  TMA producer: A and B k-blocks -> STAGES-deep shared-memory ring
//   warp 1  (elected    issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32) from the
//            lane)      128B-swizzled ring into a tensor-memory accumulator; with
//                       CTA_GROUP = 2 one instruction spans the CTA pair: 256 x BN x 16,
//                       A rows and B rows split across the two CTAs' shared memory
//   warps 2-5           epilogue: tcgen05.ld -> fp32->bf16 -> swizzled smem -> TMA store,
//                       one 32-row x 64-column box per warp per step, double-buffered,
//                       overlapping the next tile's mainloop through ACC_BUFS accumulators
//
// Shared-memory ring slots are released by tcgen05.commit onto the leader CTA's "empty"
// barriers; the leader's producer relays each release to the peer CTA with a remote
// mbarrier arrive, so no multicast form of any instruction is used.
//
// A second kernel, gemm_splitk_kernel, serves shapes with too few tiles to occupy the GPU: a
// cluster of CTAs shares one tile along K and sums its partials through distributed shared memory.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "ptx_sm100.cuh"
#include "runtime.h"

namespace b200 {
namespace {

constexpr int kBK = 64;                    // elements per k-block = one 128-byte swizzle row
constexpr int kCtaM = 128;                 // accumulator rows per CTA = tensor-memory lanes
constexpr int kAStageBytes = kCtaM * 128;  // 16 KiB
constexpr int kEpiWarps = 4;
constexpr int kEpiBoxRows = 32;
constexpr int kEpiBoxBytes = kEpiBoxRows * 128;  // 4 KiB: 32 rows x 64 bf16
constexpr int kThreads = 32 * (2 + kEpiWarps);
// Tall tiles have one group of four epilogue warps per accumulator, so that both accumulators
// of a finished tile are drained at the same time.
// (Twelve warps: registers are handed out per warp slot of the four schedulers, so ten warps
// would be budgeted like twelve anyway, 168 registers per thread; warps 2 and 3 idle.)
constexpr int threads_for(int mh) { return mh == 2 ? 384 : kThreads; }
constexpr int kMaxDst = 8;                  // copies of C one launch can write (one per GPU of a box)

// Tensor maps of every destination of C.  With one entry this is the plain GEMM; with several,
// each finished box is stored to all of them (own memory and peers' memory over NVLink), which
// is how a column shard lands in every rank's full-width C without a separate all-gather.
struct CMapSet {
    CUtensorMap m[kMaxDst];
};

constexpr int tmem_cols_for(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

// MH = 128-row halves of A a CTA works on per tile (1 or 2).  With 2, a CTA owns two
// accumulators of the same B tile: the output tile is 256 * CTA_GROUP rows tall, every B block
// loaded from L2 feeds twice the arithmetic (a quarter fewer operand bytes per flop than the
// 256 x 256 pair tile), and the two accumulators fill all 512 tensor-memory columns, so the
// epilogue overlaps the next tile's mainloop by one accumulator instead of a whole tile.
template <int BN, int STAGES, int CTA_GROUP, int ACC_BUFS, int MH = 1>
struct GemmTraits {
    static constexpr int kBRows = BN / CTA_GROUP;        // B rows this CTA loads per stage
    static constexpr int kBStageBytes = kBRows * 128;
    static constexpr int kACtaStageBytes = MH * kAStageBytes;
    static constexpr int kStageBytes = kACtaStageBytes + kBStageBytes;
    static constexpr int kRingBytes = STAGES * kStageBytes;
    // staging boxes per epilogue warp: two (store of one overlaps the fill of the other), or one
    // where there are twice the warps (their stores are off the critical path, see the epilogue)
    static constexpr int kEpiBoxesPerWarp = MH == 2 ? 1 : 2;
    static constexpr int kEpiBytes = kEpiWarps * MH * kEpiBoxesPerWarp * kEpiBoxBytes;
    static constexpr int kBarrierBytes = (2 * STAGES + 2 * ACC_BUFS) * 8 + 16;
    // +1024: the dynamic segment is only guaranteed 16-byte aligned; the ring needs 1024.
    static constexpr int kSmemBytes = kRingBytes + kEpiBytes + kBarrierBytes + 1024;
    static constexpr int kTmemCols = tmem_cols_for(ACC_BUFS * BN);
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN must be 64, 128, 192 or 256");
    static_assert(ACC_BUFS * BN <= 512, "accumulators exceed the 512 tensor-memory columns");
    static_assert(CTA_GROUP == 1 || CTA_GROUP == 2, "CTA_GROUP must be 1 or 2");
    static_assert(MH == 1 || (MH == 2 && ACC_BUFS == 2), "two A halves use one accumulator each");
    static_assert(kBRows % 8 == 0, "B rows per CTA must be a multiple of the 8-row swizzle group");
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB shared-memory limit of sm_100");
};

// tile id -> (tile row, tile column): N-tiles grouped in strips of bs_w, inside a strip the
// column index moves fastest, so concurrently running CTAs share A rows and B rows in L2.
__device__ __forceinline__ void tile_coord(int tile, int tiles_m, int tiles_n, int bs_w, int& tm,
                                           int& tn) {
    const int strip_tiles = bs_w * tiles_m;
    const int strip = tile / strip_tiles;
    const int n0 = strip * bs_w;
    const int w = min(bs_w, tiles_n - n0);
    const int r = tile - strip * strip_tiles;
    tm = r / w;
    tn = n0 + r - tm * w;
}

// ---------------------------------------------------------------- work items of a CTA group
// A CTA (pair) walks `full_waves` whole tiles (tile ids group, group + groups, ...).  The tiles
// of a ragged last wave are either handed out whole (tail_tiles of the groups take one more)
// or, with stream-K, cut along K: the tail tiles' k-blocks form one sequence that is divided
// evenly over all groups, so every group gets the same amount of work.  A group's share
// touches at most two tail tiles: the end of one (a *partial* piece: its fp32 sums go to a
// workspace slot of that group) and the beginning of the next (an *owner* piece: it starts
// at k-block 0, adds the partial pieces the following groups wrote for this tile, in group
// order, and stores the tile).  A partial piece is always a group's first tail item and an
// owner piece its last, and partial pieces wait for nobody, so owners never wait in a cycle.
struct StreamKPlan {
    int full_waves;     // whole tiles per group before the tail
    int tail_tiles;     // tiles of the ragged last wave (0: none, or not split)
    int enabled;        // 1: the tail is cut along K
    float* partials;    // [groups][CTA_GROUP][BN/4][128 rows][4] fp32 sums of partial pieces
    uint32_t* flags;    // [groups][CTA_GROUP][4 epilogue warps]: == epoch when that warp's rows are written
    uint32_t epoch;
};

struct WorkItem {
    int tile;           // tile id (rasterised by tile_coord)
    int kb_begin, kb_end;
    int kind;           // 0 whole tile, 1 owner piece (adds partials of the next groups), 2 partial piece
};

// Item `it` of `group`, or false when the group has no more work.
__device__ __forceinline__ bool work_item(const StreamKPlan& plan, int group, int groups, int num_tiles, int k_blocks,
                                          int it, WorkItem& w) {
    if (it < plan.full_waves) {
        w = WorkItem{group + it * groups, 0, k_blocks, 0};
        return true;
    }
    const int t = it - plan.full_waves;
    if (!plan.enabled) {
        // whole tail tiles to the first groups
        if (t > 0 || group >= num_tiles - plan.full_waves * groups) return false;
        w = WorkItem{plan.full_waves * groups + group, 0, k_blocks, 0};
        return true;
    }
    // this group's share [seg_begin, seg_end) of the tail's k-blocks (units of one k-block)
    const long units = static_cast<long>(plan.tail_tiles) * k_blocks;
    const long seg_begin = units * group / groups;
    const long seg_end = units * (group + 1) / groups;
    const int first_tile = static_cast<int>(seg_begin / k_blocks);
    const long first_end = static_cast<long>(first_tile + 1) * k_blocks;
    const int base = plan.full_waves * groups;
    if (t == 0) {
        if (seg_end <= seg_begin) return false;
        const int kb0 = static_cast<int>(seg_begin - static_cast<long>(first_tile) * k_blocks);
        const int kb1 = static_cast<int>((seg_end < first_end ? seg_end : first_end) - static_cast<long>(first_tile) * k_blocks);
        w = WorkItem{base + first_tile, kb0, kb1, kb0 == 0 ? 1 : 2};
        return true;
    }
    if (t == 1 && seg_end > first_end) {
        w = WorkItem{base + first_tile + 1, 0, static_cast<int>(seg_end - first_end), 1};
        return true;
    }
    return false;
}

template <int BN, int STAGES, int CTA_GROUP, int ACC_BUFS, int MH>
__global__ void __launch_bounds__(threads_for(MH), 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CMapSet tmap_c, int n_dst, int M, int N, int K, int bs_w,
                    int is_bf16, const StreamKPlan plan,
                    uint32_t* status) {
    using T = GemmTraits<BN, STAGES, CTA_GROUP, ACC_BUFS, MH>;
    constexpr int kHalfM = kCtaM * CTA_GROUP;   // rows one MMA instruction covers
    constexpr int BM = kHalfM * MH;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring_a = smem_base;
    const uint32_t ring_b = smem_base + STAGES * T::kACtaStageBytes;
    const uint32_t epi_base = smem_base + T::kRingBytes;
    const uint32_t bar_base = epi_base + T::kEpiBytes;
    const uint32_t full_bar = bar_base;                      // [STAGES] TMA -> MMA
    const uint32_t empty_bar = full_bar + STAGES * 8;        // [STAGES] MMA -> TMA
    const uint32_t accfull_bar = empty_bar + STAGES * 8;     // [ACC_BUFS] MMA -> epilogue
    const uint32_t accempty_bar = accfull_bar + ACC_BUFS * 8;  // [ACC_BUFS] epilogue -> MMA
    const uint32_t tmem_slot = accempty_bar + ACC_BUFS * 8;
    const uint32_t abort_slot = tmem_slot + 4;
    // generic pointers to the two scalar slots
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
    volatile uint32_t* abort_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CTA_GROUP == 2) ? cluster_ctarank() : 0u;
    const bool is_leader = (cta_rank == 0);
    const WaitGuard guard{abort_ptr, status};

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int b = 0; b < ACC_BUFS; ++b) {
            mbar_init(accfull_bar + 8 * b, 1);
            mbar_init(accempty_bar + 8 * b, kEpiWarps * CTA_GROUP);
        }
        *abort_ptr = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        for (int d = 0; d < n_dst; ++d) prefetch_tensormap(&tmap_c.m[d]);
    }
    if (warp == 1) {
        tmem_alloc<CTA_GROUP>(tmem_slot, T::kTmemCols);
        tmem_relinquish<CTA_GROUP>();
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) {
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    // Ragged edges cost nothing extra: TMA zero-fills loads past the end of a matrix (zero
    // rows and zero k-columns add nothing) and clips stores.
    const int tiles_m = (M + BM - 1) / BM;
    const int tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + kBK - 1) / kBK;
    const int group = blockIdx.x / CTA_GROUP;
    const int num_groups = gridDim.x / CTA_GROUP;

    constexpr int kEpiWarp0 = (MH == 2) ? 4 : 2;   // first epilogue warp
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint32_t full_leader = (CTA_GROUP == 2) ? mapa_cluster(full_bar, 0) : full_bar;
            const uint32_t empty_peer = (CTA_GROUP == 2) ? mapa_cluster(empty_bar, 1) : 0u;
            int s = 0;
            uint32_t ph = 0;
            uint32_t fills = 0;  // ring slots filled so far by this CTA
            bool ok = true;
            WorkItem item;
            for (int it = 0; ok && work_item(plan, group, num_groups, num_tiles, k_blocks, it, item); ++it) {
                int tm, tn;
                tile_coord(item.tile, tiles_m, tiles_n, bs_w, tm, tn);
                const int row_a = tm * BM + static_cast<int>(cta_rank) * kCtaM;
                const int row_b = tn * BN + static_cast<int>(cta_rank) * T::kBRows;
                for (int kb = item.kb_begin; kb < item.kb_end; ++kb) {
                    ok = mbar_wait(guard, empty_bar + 8 * s, ph ^ 1u, 0x100u + s);
                    if (!ok) break;
                    if constexpr (CTA_GROUP == 2) {
                        // The slot was released by tcgen05.commit on the leader only; pass
                        // the release on to the peer's copy of the barrier.  The first
                        // STAGES fills find the ring empty and need no release.
                        if (is_leader && fills >= static_cast<uint32_t>(STAGES)) {
                            mbar_arrive_remote(empty_peer + 8 * s);
                        }
                    }
                    if (is_leader) {
                        mbar_arrive_expect_tx(full_bar + 8 * s, T::kStageBytes * CTA_GROUP);
                    }
                    if constexpr (CTA_GROUP == 2) {
#pragma unroll
                        for (int h = 0; h < MH; ++h) {
                            tma_load_2d_pair(ring_a + s * T::kACtaStageBytes + h * kAStageBytes, &tmap_a,
                                             full_leader + 8 * s, kb * kBK, row_a + h * kHalfM);
                        }
                        tma_load_2d_pair(ring_b + s * T::kBStageBytes, &tmap_b, full_leader + 8 * s,
                                         kb * kBK, row_b);
                    } else {
#pragma unroll
                        for (int h = 0; h < MH; ++h) {
                            tma_load_2d(ring_a + s * T::kACtaStageBytes + h * kAStageBytes, &tmap_a,
                                        full_bar + 8 * s, kb * kBK, row_a + h * kHalfM);
                        }
                        tma_load_2d(ring_b + s * T::kBStageBytes, &tmap_b, full_bar + 8 * s, kb * kBK,
                                    row_b);
                    }
                    ++fills;
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------- MMA issuer
        // The whole warp runs the loop and one elected lane issues: tcgen05.mma issued from
        // warp-uniform code costs fewer issue cycles than from a single diverged lane.
        if (is_leader) {
            // operand format: bf16 (1) or fp16 (0); the accumulator is fp32 either way
            const uint32_t idesc = make_idesc_f16(kHalfM, BN, is_bf16 ? 1 : 0, 0, 0);
            int s = 0;
            uint32_t ph = 0;
            uint32_t local_tile = 0;
            bool ok = true;
            WorkItem item;
            for (int it = 0; ok && work_item(plan, group, num_groups, num_tiles, k_blocks, it, item); ++it, ++local_tile) {
                if constexpr (MH == 2) {
                    // Both accumulators belong to this tile and both are full at its end, so the
                    // two halves are skewed by kSkew k-blocks at the ends of a tile only: half 0
                    // runs its first blocks while half 1's accumulator is still being drained
                    // (half 1 then catches up on the same ring slots), and finishes its last
                    // blocks first so that its drain starts while half 1 is still computing.  In
                    // between the halves move in lockstep and no ring slot is held longer than
                    // one k-block.  (Half 0 never holds more than kSkew < STAGES slots.)
                    constexpr int kSkew = 2;
                    static_assert(kSkew < STAGES, "the lead of half 0 must fit in the ring");
                    const uint32_t acc_ph = local_tile & 1u;
                    const int n = item.kb_end - item.kb_begin;
                    const int lead = (n / 2 < kSkew) ? n / 2 : kSkew;
                    int s_back = s;   // next slot half 1 consumes (and releases); s = next slot half 0 consumes
                    // MMAs of half h on ring slot `slot`; `first`: the accumulator is overwritten
                    auto issue_half = [&](int h, int slot, bool first, bool release) {
                        const uint64_t a_desc = smem_desc_kmajor_sw128(ring_a + slot * T::kACtaStageBytes + h * kAStageBytes);
                        const uint64_t b_desc = smem_desc_kmajor_sw128(ring_b + slot * T::kBStageBytes);
                        if (elect_one()) {
#pragma unroll
                            for (int k = 0; k < kBK / 16; ++k) {
                                mma_ss<CTA_GROUP>(tmem_base + h * BN, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                                  (!first || k != 0) ? 1u : 0u);
                            }
                            if (release) mma_commit<CTA_GROUP>(empty_bar + 8 * slot);
                        }
                        __syncwarp();
                    };
                    auto front = [&](bool first) {   // half 0 takes the next slot once its data has landed
                        ok = __all_sync(0xffffffffu, mbar_wait(guard, full_bar + 8 * s, ph, 0x300u + s));
                        if (!ok) return;
                        if (first) {
                            ok = __all_sync(0xffffffffu, mbar_wait(guard, accempty_bar, acc_ph ^ 1u, 0x200u));
                            if (!ok) return;
                        }
                        tc_fence_after();
                        issue_half(0, s, first, false);
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    };
                    auto back = [&](bool first) {    // half 1 follows on a slot half 0 has used, and releases it
                        if (first) {
                            ok = __all_sync(0xffffffffu, mbar_wait(guard, accempty_bar + 8, acc_ph ^ 1u, 0x201u));
                            if (!ok) return;
                            tc_fence_after();
                        }
                        issue_half(1, s_back, first, true);
                        if (++s_back == STAGES) s_back = 0;
                    };
                    for (int kb = 0; kb < lead && ok; ++kb) front(kb == 0);
                    for (int kb = 0; kb < lead && ok; ++kb) back(kb == 0);
                    for (int kb = lead; kb < n - lead && ok; ++kb) {
                        front(kb == 0);
                        if (ok) back(kb == 0);
                    }
                    for (int kb = n - lead; kb < n && ok; ++kb) front(false);
                    if (ok && elect_one()) mma_commit<CTA_GROUP>(accfull_bar);
                    __syncwarp();
                    for (int kb = n - lead; kb < n && ok; ++kb) back(false);
                    if (ok && elect_one()) mma_commit<CTA_GROUP>(accfull_bar + 8);
                    __syncwarp();
                    continue;
                }
                const uint32_t buf = local_tile % ACC_BUFS;
                const uint32_t acc_ph = (local_tile / ACC_BUFS) & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(guard, accempty_bar + 8 * buf, acc_ph ^ 1u, 0x200u + buf));
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = item.kb_begin; kb < item.kb_end; ++kb) {
                    ok = __all_sync(0xffffffffu, mbar_wait(guard, full_bar + 8 * s, ph, 0x300u + s));
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a_desc = smem_desc_kmajor_sw128(ring_a + s * kAStageBytes);
                    const uint64_t b_desc = smem_desc_kmajor_sw128(ring_b + s * T::kBStageBytes);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k) {
                            // 16 elements of K = 32 bytes inside the swizzled row = +2 in the
                            // descriptor's 16-byte address units.
                            mma_ss<CTA_GROUP>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                              (kb != item.kb_begin || k != 0) ? 1u : 0u);
                        }
                        mma_commit<CTA_GROUP>(empty_bar + 8 * s);
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok && elect_one()) mma_commit<CTA_GROUP>(accfull_bar + 8 * buf);
                __syncwarp();
            }
        }
    } else if (warp >= kEpiWarp0) {
        // ---------------------------------------------------------------------- epilogue
        const int q = warp & 3;  // tensor-memory lane quadrant this warp may read
        const uint32_t my_epi = epi_base + (warp - kEpiWarp0) * T::kEpiBoxesPerWarp * kEpiBoxBytes;
        const int my_half = (MH == 2) ? (warp - kEpiWarp0) >> 2 : 0;   // tall tiles: the accumulator this warp drains
        const uint32_t accfull_peer = (CTA_GROUP == 2) ? mapa_cluster(accfull_bar, 1) : 0u;
        const uint32_t accempty_leader = (CTA_GROUP == 2) ? mapa_cluster(accempty_bar, 0) : accempty_bar;
        uint32_t local_tile = 0;
        uint32_t stores = 0;
        bool ok = true;
        WorkItem item;
        for (int it = 0; ok && work_item(plan, group, num_groups, num_tiles, k_blocks, it, item); ++it, ++local_tile) {
            int tm, tn;
            tile_coord(item.tile, tiles_m, tiles_n, bs_w, tm, tn);
          {
            const int h = my_half;
            const uint32_t buf = (MH == 2) ? static_cast<uint32_t>(h) : local_tile % ACC_BUFS;
            const uint32_t acc_ph = (MH == 2) ? (local_tile & 1u) : ((local_tile / ACC_BUFS) & 1u);
            // a long wait (a whole mainloop): the hardware parks the warp, see mbar_wait_limit
            ok = __all_sync(0xffffffffu, mbar_wait(guard, accfull_bar + 8 * buf, acc_ph, 0x400u + buf));
            if (!ok) break;
            if constexpr (CTA_GROUP == 2) {
                if (is_leader && ((warp - kEpiWarp0) & 3) == 0 && lane == 0) mbar_arrive_remote(accfull_peer + 8 * buf);
            }
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            const int out_row = tm * BM + h * kHalfM + static_cast<int>(cta_rank) * kCtaM + q * 32;
            // Stream-K: where this warp's 32 rows of a partial piece live in the workspace, as
            // [column group of 4][row][4 floats] so that the lanes of a warp touch 512 contiguous
            // bytes; slot = (group, CTA of the pair).
            constexpr int kSlotFloats = (BN / 4) * kCtaM * 4;
            const int row_in_cta = q * 32 + lane;
            int n_contrib = 0;
            if (item.kind == 1 && item.kb_end < k_blocks) {
                // an owner piece that stops short of the last k-block: the following groups hold the
                // rest of this tile as their first (partial) pieces.  Count them, then wait for this
                // warp's rows of each (they were started before this piece and wait for nobody).
                const long units = static_cast<long>(plan.tail_tiles) * k_blocks;
                const long tile_end = static_cast<long>(item.tile - plan.full_waves * num_groups + 1) * k_blocks;
                for (int g = group + 1; g < num_groups; ++g) {
                    ++n_contrib;
                    if (units * (g + 1) / num_groups >= tile_end) break;
                }
                for (int g = group + 1; g <= group + n_contrib && ok; ++g) {
                    const uint32_t* flag = plan.flags + (static_cast<size_t>(g) * CTA_GROUP + cta_rank) * kEpiWarps + (warp - kEpiWarp0);
                    ok = wait_flag_warp(guard, flag, plan.epoch, 0x500u);
                }
                if (!ok) break;
            }
            if constexpr (MH == 2) {
                // The next tile's mainloop waits for this accumulator: read and round all of it
                // first (128 packed registers per thread), hand it back, then stage and store.
                // (32 columns per load: 128 packed + 32 loaded registers fit the 168 of a thread)
                uint32_t packed[BN / 64][32];
#pragma unroll
                for (int c2 = 0; c2 < BN / 32; ++c2) {
                    uint32_t acc[32];
                    tmem_ld_32x32b_x32(t_row + c2 * 32, acc);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float a0 = __uint_as_float(acc[2 * i]), a1 = __uint_as_float(acc[2 * i + 1]);
                        if (is_bf16) {
                            __nv_bfloat162 v0 = __floats2bfloat162_rn(a0, a1);
                            packed[c2 >> 1][(c2 & 1) * 16 + i] = *reinterpret_cast<uint32_t*>(&v0);
                        } else {
                            __half2 v0 = __floats2half2_rn(a0, a1);
                            packed[c2 >> 1][(c2 & 1) * 16 + i] = *reinterpret_cast<uint32_t*>(&v0);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CTA_GROUP == 2) {
                        mbar_arrive_remote(accempty_leader + 8 * buf);
                    } else {
                        mbar_arrive(accempty_bar + 8 * buf);
                    }
                }
#pragma unroll
                for (int c = 0; c < BN / 64; ++c) {
                    // one staging box per warp: the previous store must have read it; this is
                    // after the hand-back, with a whole mainloop to spare
                    const uint32_t box = my_epi;
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
                    const uint32_t row_addr = box + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        st_shared_v4(row_addr + ((j ^ (lane & 7)) << 4), packed[c][4 * j], packed[c][4 * j + 1],
                                     packed[c][4 * j + 2], packed[c][4 * j + 3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        for (int d = 0; d < n_dst; ++d) tma_store_2d(&tmap_c.m[d], box, tn * BN + c * 64, out_row);
                        tma_store_commit();
                    }
                    ++stores;
                }
                continue;
            }
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
                uint32_t acc0[32], acc1[32];
                tmem_ld_32x32b_x32(t_row + c * 64, acc0);
                tmem_ld_32x32b_x32(t_row + c * 64 + 32, acc1);
                tmem_wait_ld();
                if (c == BN / 64 - 1) {
                    // Accumulator fully read: hand the buffer back to the MMA issuer.
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CTA_GROUP == 2) {
                            mbar_arrive_remote(accempty_leader + 8 * buf);
                        } else {
                            mbar_arrive(accempty_bar + 8 * buf);
                        }
                    }
                }
                if (item.kind == 2) {
                    // partial piece: park the fp32 sums for the tile's owner
                    float4* dst = reinterpret_cast<float4*>(plan.partials) +
                                  (static_cast<size_t>(group) * CTA_GROUP + cta_rank) * (kSlotFloats / 4) +
                                  static_cast<size_t>(c * 16) * kCtaM + row_in_cta;
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        dst[static_cast<size_t>(g4) * kCtaM] =
                            make_float4(__uint_as_float(acc0[4 * g4]), __uint_as_float(acc0[4 * g4 + 1]),
                                        __uint_as_float(acc0[4 * g4 + 2]), __uint_as_float(acc0[4 * g4 + 3]));
                        dst[static_cast<size_t>(8 + g4) * kCtaM] =
                            make_float4(__uint_as_float(acc1[4 * g4]), __uint_as_float(acc1[4 * g4 + 1]),
                                        __uint_as_float(acc1[4 * g4 + 2]), __uint_as_float(acc1[4 * g4 + 3]));
                    }
                    if (c == BN / 64 - 1) {
                        // every row of this warp is written: publish (release) to the owner's warp q
                        __threadfence();
                        __syncwarp();
                        if (lane == 0)
                            st_release_gpu_u32(plan.flags + (static_cast<size_t>(group) * CTA_GROUP + cta_rank) * kEpiWarps + (warp - kEpiWarp0),
                                               plan.epoch);
                    }
                    continue;
                }
                for (int g = group + 1; g <= group + n_contrib; ++g) {
                    // add the partial sums of the following groups, in group order (deterministic)
                    const float4* src = reinterpret_cast<const float4*>(plan.partials) +
                                        (static_cast<size_t>(g) * CTA_GROUP + cta_rank) * (kSlotFloats / 4) +
                                        static_cast<size_t>(c * 16) * kCtaM + row_in_cta;
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        const float4 u = ld_global_cg_f4(src + static_cast<size_t>(g4) * kCtaM);
                        const float4 v = ld_global_cg_f4(src + static_cast<size_t>(8 + g4) * kCtaM);
                        acc0[4 * g4] = __float_as_uint(__uint_as_float(acc0[4 * g4]) + u.x);
                        acc0[4 * g4 + 1] = __float_as_uint(__uint_as_float(acc0[4 * g4 + 1]) + u.y);
                        acc0[4 * g4 + 2] = __float_as_uint(__uint_as_float(acc0[4 * g4 + 2]) + u.z);
                        acc0[4 * g4 + 3] = __float_as_uint(__uint_as_float(acc0[4 * g4 + 3]) + u.w);
                        acc1[4 * g4] = __float_as_uint(__uint_as_float(acc1[4 * g4]) + v.x);
                        acc1[4 * g4 + 1] = __float_as_uint(__uint_as_float(acc1[4 * g4 + 1]) + v.y);
                        acc1[4 * g4 + 2] = __float_as_uint(__uint_as_float(acc1[4 * g4 + 2]) + v.z);
                        acc1[4 * g4 + 3] = __float_as_uint(__uint_as_float(acc1[4 * g4 + 3]) + v.w);
                    }
                }
                uint32_t packed[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float a0 = __uint_as_float(acc0[2 * i]), a1 = __uint_as_float(acc0[2 * i + 1]);
                    const float b0 = __uint_as_float(acc1[2 * i]), b1 = __uint_as_float(acc1[2 * i + 1]);
                    if (is_bf16) {
                        __nv_bfloat162 v0 = __floats2bfloat162_rn(a0, a1);
                        __nv_bfloat162 v1 = __floats2bfloat162_rn(b0, b1);
                        packed[i] = *reinterpret_cast<uint32_t*>(&v0);
                        packed[16 + i] = *reinterpret_cast<uint32_t*>(&v1);
                    } else {
                        __half2 v0 = __floats2half2_rn(a0, a1);
                        __half2 v1 = __floats2half2_rn(b0, b1);
                        packed[i] = *reinterpret_cast<uint32_t*>(&v0);
                        packed[16 + i] = *reinterpret_cast<uint32_t*>(&v1);
                    }
                }
                const uint32_t box = my_epi + (stores & 1u) * kEpiBoxBytes;
                // The store issued two steps ago read this box; wait until it has.
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                const uint32_t row_addr = box + lane * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    st_shared_v4(row_addr + ((j ^ (lane & 7)) << 4), packed[4 * j], packed[4 * j + 1],
                                 packed[4 * j + 2], packed[4 * j + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    for (int d = 0; d < n_dst; ++d) tma_store_2d(&tmap_c.m[d], box, tn * BN + c * 64, out_row);
                    tma_store_commit();
                }
                ++stores;
            }
          }
        }
        if (lane == 0) tma_store_wait_all<0>();
    }

    // ------------------------------------------------------------------------- teardown
    if (*abort_ptr != 0) {
        // A wait gave up: let copies and MMAs already in flight retire before the shared
        // and tensor memory they target is released.
        for (int i = 0; i < 64; ++i) __nanosleep(100000);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) {
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc<CTA_GROUP>(tmem_base, T::kTmemCols);
    }
}

// ------------------------------------------------------------------------- split-K kernel
// For shapes with too few output tiles to occupy the GPU (M = 128 with a long K: the problem
// is then bound by reading B once from HBM, and only CTAs that are loading count).  A cluster
// of SPLIT CTAs shares one 128 x BN output tile: CTA r accumulates k-blocks
// [r*kb/SPLIT, (r+1)*kb/SPLIT) in tensor memory, parks its fp32 partial tile in its own shared
// memory (over the drained ring), and after a cluster barrier each CTA sums a 128/SPLIT-row
// band of all partials through distributed shared memory, in rank order (deterministic),
// rounds once and stores to C.  No workspace in global memory, no second kernel.
struct CPtrSet {
    void* p[kMaxDst];
};

template <int BN, int STAGES>
struct SplitKTraits {
    static constexpr int kBStageBytes = BN * 128;
    static constexpr int kStageBytes = kAStageBytes + kBStageBytes;
    static constexpr int kRingBytes = STAGES * kStageBytes;
    static constexpr int kPartialBytes = kCtaM * BN * 4;   // [BN/4][128 rows][4 floats]
    static constexpr int kBarrierBytes = (2 * STAGES + 1) * 8 + 16;
    static constexpr int kSmemBytes = kRingBytes + kBarrierBytes + 1024;
    static constexpr int kTmemCols = tmem_cols_for(BN);
    static_assert(BN == 64 || BN == 128 || BN == 256, "split-K tiles are 128 x 64, 128 x 128 or 128 x 256");
    static_assert(kPartialBytes <= kRingBytes, "the partial tile must fit over the ring");
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB shared-memory limit of sm_100");
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CPtrSet c_list, int n_dst, int64_t ldc, int M, int N, int K,
                   int split, int is_bf16, uint32_t* status) {
    using T = SplitKTraits<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring_a = smem_base;
    const uint32_t ring_b = smem_base + STAGES * kAStageBytes;
    const uint32_t partial = smem_base;                       // over the ring, after the mainloop
    const uint32_t bar_base = smem_base + T::kRingBytes;
    const uint32_t full_bar = bar_base;                       // [STAGES] TMA -> MMA
    const uint32_t empty_bar = full_bar + STAGES * 8;         // [STAGES] MMA -> TMA
    const uint32_t accfull_bar = empty_bar + STAGES * 8;      // MMA -> epilogue
    const uint32_t tmem_slot = accfull_bar + 8;
    const uint32_t abort_slot = tmem_slot + 4;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
    volatile uint32_t* abort_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));
    const WaitGuard guard{abort_ptr, status};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());     // = blockIdx.x % split
    const int tile = static_cast<int>(blockIdx.x) / split;
    const int tiles_n = (N + BN - 1) / BN;
    const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
    // k-blocks of this rank: an even share, the first (total % split) ranks take one more
    const int kb_total = (K + kBK - 1) / kBK;
    const int kb_base = kb_total / split, kb_rem = kb_total - kb_base * split;
    const int kb_begin = rank * kb_base + min(rank, kb_rem);
    const int kb_count = kb_base + (rank < kb_rem ? 1 : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        mbar_init(accfull_bar, 1);
        *abort_ptr = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, T::kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < kb_count; ++kb) {
                if (!mbar_wait(guard, empty_bar + 8 * s, ph ^ 1u, 0x2100u + s)) break;
                mbar_arrive_expect_tx(full_bar + 8 * s, T::kStageBytes);
                tma_load_2d(ring_a + s * kAStageBytes, &tmap_a, full_bar + 8 * s, (kb_begin + kb) * kBK, tm * kCtaM);
                tma_load_2d(ring_b + s * T::kBStageBytes, &tmap_b, full_bar + 8 * s, (kb_begin + kb) * kBK, tn * BN);
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(kCtaM, BN, is_bf16 ? 1 : 0, 0, 0);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int kb = 0; kb < kb_count; ++kb) {
            ok = __all_sync(0xffffffffu, mbar_wait(guard, full_bar + 8 * s, ph, 0x2300u + s));
            if (!ok) break;
            tc_fence_after();
            const uint64_t a_desc = smem_desc_kmajor_sw128(ring_a + s * kAStageBytes);
            const uint64_t b_desc = smem_desc_kmajor_sw128(ring_b + s * T::kBStageBytes);
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)
                    mma_ss<1>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                mma_commit<1>(empty_bar + 8 * s);
            }
            __syncwarp();
            if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok && kb_count > 0 && elect_one()) mma_commit<1>(accfull_bar);
        __syncwarp();
    } else {
        // park the fp32 partial tile: thread = row, 4 columns per 16-byte store, column-group major
        const int q = warp & 3;
        const int row = q * 32 + lane;
        bool ok = true;
        if (kb_count > 0) {
            ok = __all_sync(0xffffffffu, mbar_wait(guard, accfull_bar, 0, 0x2400u));
            tc_fence_after();
        }
        if (ok) {
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t acc[32];
                if (kb_count > 0) {
                    tmem_ld_32x32b_x32(t_row + c * 32, acc);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int x = 0; x < 32; ++x) acc[x] = 0u;
                }
#pragma unroll
                for (int g = 0; g < 8; ++g)
                    st_shared_v4(partial + (c * 8 + g) * (kCtaM * 16) + row * 16, acc[4 * g], acc[4 * g + 1],
                                 acc[4 * g + 2], acc[4 * g + 3]);
            }
        }
    }

    // every partial of the cluster is in place
    tc_fence_before();
    __syncwarp();
    cluster_arrive();
    cluster_wait();

    if (warp >= 2 && *abort_ptr == 0) {
        const int rows_per = kCtaM / split;
        const int t = threadIdx.x - 64;
        for (int idx = t; idx < rows_per * (BN / 4); idx += kEpiWarps * 32) {
            const int cg = idx / rows_per;
            const int row = rank * rows_per + (idx - cg * rows_per);
            const uint32_t local = partial + cg * (kCtaM * 16) + row * 16;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            for (int r = 0; r < split; ++r) {
                float a, b, c, d;
                ld_shared_cluster_v4(mapa_cluster(local, static_cast<uint32_t>(r)), a, b, c, d);
                s0 += a; s1 += b; s2 += c; s3 += d;
            }
            const int grow = tm * kCtaM + row, gcol = tn * BN + cg * 4;
            if (grow < M && gcol < N) {
                uint2 out;
                if (is_bf16) {
                    __nv_bfloat162 v0 = __floats2bfloat162_rn(s0, s1), v1 = __floats2bfloat162_rn(s2, s3);
                    out.x = *reinterpret_cast<uint32_t*>(&v0);
                    out.y = *reinterpret_cast<uint32_t*>(&v1);
                } else {
                    __half2 v0 = __floats2half2_rn(s0, s1), v1 = __floats2half2_rn(s2, s3);
                    out.x = *reinterpret_cast<uint32_t*>(&v0);
                    out.y = *reinterpret_cast<uint32_t*>(&v1);
                }
                for (int d = 0; d < n_dst; ++d)
                    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(c_list.p[d]) + static_cast<int64_t>(grow) * ldc + gcol) = out;
            }
        }
    }

    // ------------------------------------------------------------------------- teardown
    if (*abort_ptr != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(100000);
    }
    // no CTA may exit (and release its shared memory) while a peer still reads its partial
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc<1>(tmem_base, T::kTmemCols);
    }
}

// ------------------------------------------------------------------------- host launcher
// Workspaces of stream-K launches: fp32 partial tiles and their flags.  Kept in a small
// per-device pool; each carries the stream and the event of the last launch that used it.  A
// launch takes the one last used on its own stream (stream order already keeps those
// kernels apart), else the first one whose event has completed, else a new one, so launches
// that can overlap never share a workspace.  Flags are compared with a per-
// workspace epoch that grows with every launch, so they never need clearing.
struct StreamKWorkspace {
    float* partials = nullptr;
    uint32_t* flags = nullptr;
    size_t partial_bytes = 0, flag_bytes = 0;
    uint32_t epoch = 0;
    cudaEvent_t done = nullptr;
    cudaStream_t last_stream = nullptr;
    bool in_use = false;      // taken by a launch that has not recorded its event yet
};
constexpr int kMaxWorkspaces = 8;
StreamKWorkspace g_workspaces[kMaxDevices][kMaxWorkspaces];
std::mutex g_workspace_mutex;

StreamKWorkspace* acquire_stream_k_workspace(int device, cudaStream_t stream, size_t partial_bytes,
                                             size_t flag_bytes) {
    std::lock_guard<std::mutex> lock(g_workspace_mutex);
    StreamKWorkspace* free_slot = nullptr;
    for (int i = 0; i < kMaxWorkspaces; ++i) {
        StreamKWorkspace& w = g_workspaces[device][i];
        if (!w.in_use && w.partials != nullptr && w.last_stream == stream && w.partial_bytes >= partial_bytes &&
            w.flag_bytes >= flag_bytes) {
            w.in_use = true;
            return &w;
        }
    }
    for (int i = 0; i < kMaxWorkspaces; ++i) {
        StreamKWorkspace& w = g_workspaces[device][i];
        if (w.in_use) continue;
        if (w.partials == nullptr) {
            if (free_slot == nullptr) free_slot = &w;
            continue;
        }
        if (cudaEventQuery(w.done) != cudaSuccess) {
            (void)cudaGetLastError();   // cudaErrorNotReady: still running
            continue;
        }
        if (w.partial_bytes < partial_bytes || w.flag_bytes < flag_bytes) {
            // idle but too small: replace it
            cudaFree(w.partials);
            cudaFree(w.flags);
            w.partials = nullptr;
            w.flags = nullptr;
            if (free_slot == nullptr) free_slot = &w;
            continue;
        }
        w.in_use = true;
        return &w;
    }
    if (free_slot == nullptr) {
        fail(B200_ECUDA, "more than %d stream-K launches in flight on device %d", kMaxWorkspaces, device);
        return nullptr;
    }
    StreamKWorkspace& w = *free_slot;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&w.partials), partial_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&w.flags), flag_bytes);
    if (e == cudaSuccess) e = cudaMemset(w.flags, 0, flag_bytes);
    if (e == cudaSuccess && w.done == nullptr) e = cudaEventCreateWithFlags(&w.done, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        fail(B200_ECUDA, "stream-K workspace (%zu bytes): %s", partial_bytes + flag_bytes, cudaGetErrorString(e));
        if (w.partials) cudaFree(w.partials);
        if (w.flags) cudaFree(w.flags);
        w.partials = nullptr;
        w.flags = nullptr;
        return nullptr;
    }
    w.partial_bytes = partial_bytes;
    w.flag_bytes = flag_bytes;
    w.epoch = 0;
    w.in_use = true;
    return &w;
}

void release_stream_k_workspace(StreamKWorkspace* w, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_workspace_mutex);
    (void)cudaEventRecord(w->done, stream);
    w->last_stream = stream;
    w->in_use = false;
}

// Whether a launch with this many tiles, CTA groups and k-blocks cuts its last wave along K.
std::atomic<int> g_stream_k_mode{0};   // b200_gemm_set_stream_k: 0 = off (default), 1 = on
bool wants_stream_k(int num_tiles, int groups, int k_blocks) {
    if (g_stream_k_mode.load(std::memory_order_relaxed) == 0) return false;
    const int tail = num_tiles % groups;
    return tail > 0 && tail * 10 <= groups * 9 && k_blocks >= 16 && num_tiles * 2 >= groups;
}

using LaunchFn = int (*)(const DeviceInfo*, const b200_gemm_config&, int, int, int, const void*,
                         int64_t, const void*, int64_t, void* const*, int, int64_t, bool, cudaStream_t);

template <int BN, int STAGES, int CTA_GROUP, int ACC_BUFS, int MH = 1>
int launch_gemm(const DeviceInfo* dev, const b200_gemm_config& cfg, int M, int N, int K,
                const void* A, int64_t lda, const void* B, int64_t ldb, void* const* C_list, int n_dst,
                int64_t ldc, bool is_bf16, cudaStream_t stream) {
    using T = GemmTraits<BN, STAGES, CTA_GROUP, ACC_BUFS, MH>;
    auto kernel = gemm_bf16_tn_kernel<BN, STAGES, CTA_GROUP, ACC_BUFS, MH>;
    constexpr int BM = kCtaM * CTA_GROUP * MH;

    CUtensorMap tmap_a, tmap_b;
    CMapSet tmap_c;
    std::memset(&tmap_c, 0, sizeof(tmap_c));
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
        const uint32_t box[2] = {kBK, kCtaM};
        if (int rc = encode_tmap_2byte(&tmap_a, A, 2, dims, strides, box, true)) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
        const uint32_t box[2] = {kBK, static_cast<uint32_t>(T::kBRows)};
        if (int rc = encode_tmap_2byte(&tmap_b, B, 2, dims, strides, box, true)) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldc) * 2};
        const uint32_t box[2] = {64, kEpiBoxRows};
        for (int d = 0; d < n_dst; ++d) {
            if (int rc = encode_tmap_2byte(&tmap_c.m[d], C_list[d], 2, dims, strides, box, true)) return rc;
        }
    }

    // Set once per (kernel, device); the reference sets it on every call
    // (gemm/gemm_cute.hpp:339-341).
    static bool attr_done[kMaxDevices] = {};
    if (int rc = set_smem_once(kernel, T::kSmemBytes, dev->device, attr_done, cfg.name)) return rc;

    const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int k_blocks = (K + kBK - 1) / kBK;
    int groups = dev->sm_count / CTA_GROUP;

    // Ragged last wave: cut its tiles along K over all groups (stream-K) when that saves more
    // than the fix-up costs -- at least a tenth of a tile time per group, tiles long enough to
    // amortise parking and re-reading a partial tile, and not the few-tile regime the cluster
    // split-K kernel serves.  The workspace comes from a per-device pool: a launch takes one
    // whose previous launch has finished (or a new one), so overlapping launches never share.
    StreamKPlan plan{};
    // (tiles with two accumulators per CTA are never cut: both accumulators are in use)
    const bool stream_k = MH == 1 && dev->may_allocate && wants_stream_k(num_tiles, groups, k_blocks);
    if (!stream_k && groups > num_tiles) groups = num_tiles;
    plan.full_waves = num_tiles / groups;
    plan.tail_tiles = num_tiles % groups;
    StreamKWorkspace* ws = nullptr;
    if (stream_k) {
        const size_t slot_bytes = static_cast<size_t>(BN) * kCtaM * sizeof(float);
        const size_t partial_bytes = static_cast<size_t>(groups) * CTA_GROUP * slot_bytes;
        const size_t flag_bytes = static_cast<size_t>(groups) * CTA_GROUP * kEpiWarps * sizeof(uint32_t);
        ws = acquire_stream_k_workspace(dev->device, stream, partial_bytes, flag_bytes);
        if (ws == nullptr) return B200_ECUDA;
        plan.enabled = 1;
        plan.partials = ws->partials;
        plan.flags = ws->flags;
        plan.epoch = ++ws->epoch;
    }

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(groups * CTA_GROUP), 1, 1);
    lc.blockDim = dim3(threads_for(MH), 1, 1);
    lc.dynamicSmemBytes = T::kSmemBytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTA_GROUP;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, kernel, tmap_a, tmap_b, tmap_c, n_dst, M, N, K, cfg.bs_w,
                                       is_bf16 ? 1 : 0, plan, dev->status);
    if (ws != nullptr) release_stream_k_workspace(ws, stream);
    if (e != cudaSuccess) return fail(B200_ECUDA, "launch of %s failed: %s", cfg.name, cudaGetErrorString(e));
    return B200_OK;
}

template <int BN, int STAGES>
int launch_gemm_splitk(const DeviceInfo* dev, const b200_gemm_config& cfg, int M, int N, int K, const void* A,
                       int64_t lda, const void* B, int64_t ldb, void* const* C_list, int n_dst, int64_t ldc,
                       bool is_bf16, cudaStream_t stream) {
    using T = SplitKTraits<BN, STAGES>;
    auto kernel = gemm_splitk_kernel<BN, STAGES>;
    const int split = cfg.split_k;
    if ((K + kBK - 1) / kBK < split)
        return fail(B200_ESHAPE, "%s: K=%d has fewer 64-element blocks than the %d-way split", cfg.name, K, split);

    CUtensorMap tmap_a, tmap_b;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
        const uint32_t box[2] = {kBK, kCtaM};
        if (int rc = encode_tmap_2byte(&tmap_a, A, 2, dims, strides, box, true)) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
        const uint32_t box[2] = {kBK, static_cast<uint32_t>(BN)};
        if (int rc = encode_tmap_2byte(&tmap_b, B, 2, dims, strides, box, true)) return rc;
    }
    CPtrSet c_list;
    std::memset(&c_list, 0, sizeof(c_list));
    for (int d = 0; d < n_dst; ++d) {
        if ((reinterpret_cast<uintptr_t>(C_list[d]) & 7u) != 0)
            return fail(B200_EINVAL, "%s: C must be 8-byte aligned", cfg.name);
        c_list.p[d] = C_list[d];
    }

    static bool attr_done[kMaxDevices] = {};
    if (int rc = set_smem_once(kernel, T::kSmemBytes, dev->device, attr_done, cfg.name)) return rc;
    const long tiles = static_cast<long>((M + kCtaM - 1) / kCtaM) * ((N + BN - 1) / BN);
    if (tiles * split > 0x7fffffffL) return fail(B200_ESHAPE, "%s: too many tiles", cfg.name);

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
    lc.blockDim = dim3(kThreads, 1, 1);
    lc.dynamicSmemBytes = T::kSmemBytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(split);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, kernel, tmap_a, tmap_b, c_list, n_dst, ldc, M, N, K, split,
                                       is_bf16 ? 1 : 0, dev->status);
    if (e != cudaSuccess) return fail(B200_ECUDA, "launch of %s failed: %s", cfg.name, cudaGetErrorString(e));
    return B200_OK;
}

// Clusters of `split` CTAs of this kernel the current device can hold at once (a cluster must
// fit inside one GPC, so 8-CTA clusters leave SMs unused), or 0 when it cannot be asked.
template <int BN, int STAGES>
int splitk_active_clusters(int split, int sm_count) {
    using T = SplitKTraits<BN, STAGES>;
    static int cached[9] = {};
    if (split < 1 || split > 8) return 0;
    if (cached[split] != 0) return cached[split] > 0 ? cached[split] : 0;
    auto kernel = gemm_splitk_kernel<BN, STAGES>;
    int n = 0;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(split * sm_count), 1, 1);
    lc.blockDim = dim3(kThreads, 1, 1);
    lc.dynamicSmemBytes = T::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(split);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kernel, &lc) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();  // no usable device: the caller falls back to an estimate
        cached[split] = -1;
        return 0;
    }
    cached[split] = n;
    return n;
}

using ClustersFn = int (*)(int, int);

struct Entry {
    b200_gemm_config cfg;
    LaunchFn launch;
    ClustersFn active_clusters;   // split-K entries only
};

#define B200_GEMM_CONFIG(NAME, BN, STAGES, CTA_GROUP, ACC_BUFS, BS_W)                                  \
    Entry{b200_gemm_config{NAME, kCtaM * CTA_GROUP, BN, kBK, STAGES, CTA_GROUP, ACC_BUFS, BS_W,        \
                           GemmTraits<BN, STAGES, CTA_GROUP, ACC_BUFS>::kSmemBytes,                    \
                           GemmTraits<BN, STAGES, CTA_GROUP, ACC_BUFS>::kTmemCols, 1},                 \
          &launch_gemm<BN, STAGES, CTA_GROUP, ACC_BUFS>, nullptr},
#define B200_GEMM_TALL_CONFIG(NAME, BN, STAGES, BS_W)                                                  \
    Entry{b200_gemm_config{NAME, kCtaM * 4, BN, kBK, STAGES, 2, 2, BS_W,                               \
                           GemmTraits<BN, STAGES, 2, 2, 2>::kSmemBytes,                                \
                           GemmTraits<BN, STAGES, 2, 2, 2>::kTmemCols, 1},                             \
          &launch_gemm<BN, STAGES, 2, 2, 2>, nullptr},
#define B200_GEMM_SPLITK_CONFIG(NAME, BN, STAGES, SPLIT_K)                                             \
    Entry{b200_gemm_config{NAME, kCtaM, BN, kBK, STAGES, 1, 1, 1, SplitKTraits<BN, STAGES>::kSmemBytes, \
                           SplitKTraits<BN, STAGES>::kTmemCols, SPLIT_K},                              \
          &launch_gemm_splitk<BN, STAGES>, &splitk_active_clusters<BN, STAGES>},

const Entry kEntries[] = {
#include "generated/gemm_configs.inc"
};
#undef B200_GEMM_CONFIG
#undef B200_GEMM_TALL_CONFIG
#undef B200_GEMM_SPLITK_CONFIG

constexpr int kNumEntries = static_cast<int>(sizeof(kEntries) / sizeof(kEntries[0]));

// ---------------------------------------------------------------- allocation-free variant
// Scratch for b200_gemm_bf16_tn_noalloc: the block the kernel writes its status word into
// when a bounded wait gives up.  It lives in the library image, so every GPU that loads
// the library holds these 256 bytes until the process exits, and no call has to allocate.
// The name below is only a host-side stand-in for the symbol: host code must ask the
// runtime for the device address (cudaGetSymbolAddress) and may not pass the name itself.
constexpr size_t kNoAllocScratchBytes = 256;   // maximum scratch the variant can serve
constexpr size_t kStatusBlockBytes = 256;      // what one GEMM launch needs
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct NoAllocDevice {
    bool ready = false;
    DeviceInfo info;
};
NoAllocDevice g_noalloc_devices[64];
std::mutex g_noalloc_mutex;

// Once per device, with that device current: read the device facts the launcher needs
// and resolve the device address of the scratch array.  Calls nothing that allocates.
const DeviceInfo* noalloc_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        fail(B200_ENODEVICE, "cudaGetDevice failed or device index out of range: %s", cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocDevice& slot = g_noalloc_devices[dev];
    if (slot.ready) return &slot.info;
    DeviceInfo info;
    info.device = dev;
    if ((e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) {
        fail(B200_ECUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    if (info.cc_major != 10) {
        fail(B200_ENODEVICE, "device %d has compute capability %d.x; this library contains sm_100a code only", dev,
             info.cc_major);
        return nullptr;
    }
    void* scratch = nullptr;
    e = cudaGetSymbolAddress(&scratch, g_noalloc_scratch);
    if (e != cudaSuccess || scratch == nullptr) {
        fail(B200_ECUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
        return nullptr;
    }
    info.status = static_cast<uint32_t*>(scratch);
    info.may_allocate = false;
    slot.info = info;
    slot.ready = true;
    return &slot.info;
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_gemm_num_configs(void) { return b200::kNumEntries; }

const b200_gemm_config* b200_gemm_get_config(int idx) {
    if (idx < 0 || idx >= b200::kNumEntries) return nullptr;
    return &b200::kEntries[idx].cfg;
}

int b200_gemm_find_config(const char* name) {
    if (name == nullptr) return -1;
    for (int i = 0; i < b200::kNumEntries; ++i) {
        if (std::strcmp(name, b200::kEntries[i].cfg.name) == 0) return i;
    }
    return -1;
}

int b200_gemm_set_stream_k(int mode) {
    if (mode != 0 && mode != 1) return b200::fail(B200_EINVAL, "stream-K mode must be 0 or 1 (got %d)", mode);
    b200::g_stream_k_mode.store(mode, std::memory_order_relaxed);
    return B200_OK;
}

int b200_gemm_uses_stream_k(int config, int M, int N, int K) {
    using namespace b200;
    if (config < 0 || config >= kNumEntries || M <= 0 || N <= 0 || K <= 0) return 0;
    const b200_gemm_config& c = kEntries[config].cfg;
    if (c.split_k > 1 || c.bm > 128 * c.cta_group) return 0;   // split-K and tall tiles are never cut
    int sms = current_sm_count();
    if (sms <= 0) sms = 148;
    const int tiles = ((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
    return wants_stream_k(tiles, sms / c.cta_group, (K + c.bk - 1) / c.bk) ? 1 : 0;
}

int b200_gemm_default_config(int M, int N, int K) {
    // Cost model in microseconds, fitted to measurements on a B200:
    //   waves over the SMs  x  k-blocks per CTA  x  time of one k-block  +  fixed costs.
    // One k-block of a 128 x BN CTA tile takes 0.22 / 0.29 / 0.36 / 0.43 us of tensor work for
    // BN = 64 / 128 / 192 / 256 (a 128 x N x 16 MMA costs >= ~74 cycles whatever N is;
    // 8192^3 runs at 0.67 / 1.11 / 1.55 PFLOP/s with BN = 64 / 128 / 256), a CTA pair
    // saves ~6 % at BN = 256.  Where the tiles do not fill the GPU the loads bound it instead:
    // ~95 GB/s per CTA, ~11.5 TB/s from L2 in total.  Split-K pays ~8 us for the cluster
    // epilogue (12 us for 8-CTA clusters), and its waves are counted in clusters the device
    // can hold at once.  Work on a ragged edge is paid like any other.
    if (M <= 0 || N <= 0 || K <= 0) return -1;
    // SMs of the current device; without a usable device (host-side planning) a B200's 148.
    int sms = b200::current_sm_count();
    if (sms <= 0) sms = 148;
    int best = -1;
    double best_cost = 0.0;
    for (int i = 0; i < b200::kNumEntries; ++i) {
        const b200_gemm_config& c = b200::kEntries[i].cfg;
        const long tiles = static_cast<long>((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
        const long kb = (K + c.bk - 1) / c.bk;
        if (c.split_k > 1 && (tiles >= sms || kb / c.split_k < 16)) continue;  // see b200dl.h
        long slots = sms / c.cta_group;   // CTA pairs or CTAs resident at once
        if (c.split_k > 1) {
            const int held = b200::kEntries[i].active_clusters(c.split_k, sms);
            // a cluster must fit inside one GPC, so large clusters leave SMs unused
            slots = held > 0 ? held : (c.split_k == 8 ? sms / 10 : (sms - 4) / c.split_k);
        }
        const long waves = (tiles + slots - 1) / slots;
        const long ctas = tiles * c.cta_group * c.split_k;
        const long active = ctas < sms ? ctas : sms;
        double t_kb = c.bn >= 256 ? (c.cta_group == 2 ? 0.40 : 0.43) : c.bn >= 192 ? 0.36 : c.bn >= 128 ? 0.29 : 0.22;
        // Tall tiles (two accumulators per CTA): twice the work per k-block at a quarter fewer
        // operand bytes per flop, which under the power cap is worth 3-7 % on long problems
        // (measured: 8192^3 +7 %, K = 4096 shapes +1-3 %); their epilogue overlaps less.
        const int halves = c.bm / (128 * c.cta_group);
        if (halves == 2) t_kb *= 2.0 * 0.97;
        // (only where the operands do not sit in L2: 2048^3 reads its 16 MB from L2 at more than that)
        const double operand_mb = 2.0 * (static_cast<double>(M) + N) * K / 1e6;
        if ((ctas < sms || c.split_k > 1) && operand_mb > 64.0) {
            const double bytes = (128.0 + c.bn / c.cta_group) * 128.0;                 // A and B rows of one k-block
            const double gbs = 95.0 < 11500.0 / active ? 95.0 : 11500.0 / active;       // per CTA
            const double t_mem = bytes / (gbs * 1e3);
            if (t_mem > t_kb) t_kb = t_mem;
        }
        const double kb_per_cta = static_cast<double>((kb + c.split_k - 1) / c.split_k);
        // persistent kernels overlap all but the last epilogue with the next tile's mainloop
        const double fixed = c.split_k > 1 ? (c.split_k == 8 ? 12.0 : 8.0 + 0.25 * c.split_k)
                                           : (halves == 2 ? 4.0 + 0.8 * (waves - 1)
                                              : c.acc_bufs > 1 ? 4.0 : 4.0 + 1.5 * (waves - 1)) +
                                                 // the pair handshake per tile shows on latency-bound problems
                                                 // (2048^3: 64 pair tiles 18.7 us, 128 single-CTA tiles 16.7 us)
                                                 ((c.cta_group == 2 && tiles < sms / 2) ? 2.5 : 0.0);
        double cost = waves * kb_per_cta * t_kb + fixed;
        // ties: deeper ring; strip width 8 (16 for tall tiles), fastest measured on 8192^3
        cost *= 1.0 - 0.0005 * c.stages - (c.bs_w == (halves == 2 ? 16 : 8) ? 0.0002 : 0.0);
        if (best < 0 || cost < best_cost) {
            best_cost = cost;
            best = i;
        }
    }
    return best;
}

}  // extern "C"

namespace b200 {
namespace {

// Argument checks shared by every GEMM entry point.  On success *entry is the config's table
// entry; the device-dependent check (shared memory) is done by the caller, which knows
// which device record it uses.
int check_gemm_args(int config, int M, int N, int K, const void* A, int64_t lda, const void* B, int64_t ldb,
                    void* const* C_list, int n_dst, int64_t ldc, const Entry** entry) {
    if (config < 0 || config >= kNumEntries) return fail(B200_EINVAL, "unknown GEMM config index %d", config);
    if (A == nullptr || B == nullptr || C_list == nullptr) return fail(B200_EINVAL, "null matrix pointer");
    if (n_dst < 1 || n_dst > kMaxDst) return fail(B200_EINVAL, "n_dst must be 1..%d (got %d)", kMaxDst, n_dst);
    for (int d = 0; d < n_dst; ++d)
        if (C_list[d] == nullptr) return fail(B200_EINVAL, n_dst == 1 ? "null matrix pointer" : "destination %d is null", d);
    if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ESHAPE, "M, N, K must be positive (got %d %d %d)", M, N, K);
    if (N % 8 != 0) return fail(B200_ESHAPE, "N must be a multiple of 8 (TMA stores clip at 16-byte granularity), got %d", N);
    if (lda < K || ldb < K || ldc < N || lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0) {
        return fail(B200_EINVAL, "leading dimensions must be >= the row length and multiples of 8 (lda %lld ldb %lld ldc %lld)",
                    static_cast<long long>(lda), static_cast<long long>(ldb), static_cast<long long>(ldc));
    }
    *entry = &kEntries[config];
    return B200_OK;
}

int run_gemm(const DeviceInfo* dev, const Entry& e, int M, int N, int K, const void* A, int64_t lda, const void* B,
             int64_t ldb, void* const* C_list, int n_dst, int64_t ldc, bool is_bf16, void* stream) {
    if (dev == nullptr) return B200_ENODEVICE;
    if (e.cfg.smem_bytes > dev->max_smem_optin) {
        return fail(B200_ESHAPE, "%s needs %d bytes of shared memory, device allows %d", e.cfg.name, e.cfg.smem_bytes,
                    dev->max_smem_optin);
    }
    return e.launch(dev, e.cfg, M, N, K, A, lda, B, ldb, C_list, n_dst, ldc, is_bf16, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_gemm_bf16_tn(int config, int M, int N, int K, const void* A, int64_t lda, const void* B,
                      int64_t ldb, void* C, int64_t ldc, void* stream) {
    using namespace b200;
    const Entry* e = nullptr;
    if (int rc = check_gemm_args(config, M, N, K, A, lda, B, ldb, &C, 1, ldc, &e)) return rc;
    return run_gemm(current_device(), *e, M, N, K, A, lda, B, ldb, &C, 1, ldc, true, stream);
}

int b200_gemm_f16_tn(int config, int M, int N, int K, const void* A, int64_t lda, const void* B,
                     int64_t ldb, void* C, int64_t ldc, void* stream) {
    using namespace b200;
    const Entry* e = nullptr;
    if (int rc = check_gemm_args(config, M, N, K, A, lda, B, ldb, &C, 1, ldc, &e)) return rc;
    return run_gemm(current_device(), *e, M, N, K, A, lda, B, ldb, &C, 1, ldc, false, stream);
}

int b200_gemm_bf16_tn_scatter(int config, int M, int N, int K, const void* A, int64_t lda, const void* B,
                              int64_t ldb, void* const* C_list, int n_dst, int64_t ldc, void* stream) {
    using namespace b200;
    const Entry* e = nullptr;
    if (int rc = check_gemm_args(config, M, N, K, A, lda, B, ldb, C_list, n_dst, ldc, &e)) return rc;
    return run_gemm(current_device(), *e, M, N, K, A, lda, B, ldb, C_list, n_dst, ldc, true, stream);
}

int b200_gemm_bf16_tn_noalloc(int config, int M, int N, int K, const void* A, int64_t lda, const void* B,
                              int64_t ldb, void* C, int64_t ldc, void* stream) {
    using namespace b200;
    const Entry* e = nullptr;
    if (int rc = check_gemm_args(config, M, N, K, A, lda, B, ldb, &C, 1, ldc, &e)) return rc;
    // Scratch this launch needs against what the built-in array can serve.
    const size_t scratch_needed = kStatusBlockBytes;
    if (scratch_needed > kNoAllocScratchBytes) {
        return fail(B200_ESHAPE, "%s on %dx%dx%d needs %zu bytes of scratch; the allocation-free entry point serves at most %zu",
                    e->cfg.name, M, N, K, scratch_needed, kNoAllocScratchBytes);
    }
    const DeviceInfo* dev = noalloc_device();
    if (dev == nullptr) return B200_ENODEVICE;
    // The array keeps whatever the previous call left; the status word must start at zero
    // for this launch's record.  Ordered on the caller's stream, ahead of the kernel.
    cudaError_t ce = cudaMemsetAsync(dev->status, 0, kStatusBlockBytes, static_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return fail(B200_ECUDA, "clearing the scratch block failed: %s", cudaGetErrorString(ce));
    return run_gemm(dev, *e, M, N, K, A, lda, B, ldb, &C, 1, ldc, true, stream);
}

int b200_gemm_noalloc_status(uint32_t* code) {
    using namespace b200;
    if (code == nullptr) return fail(B200_EINVAL, "code is null");
    const DeviceInfo* dev = noalloc_device();
    if (dev == nullptr) return B200_ENODEVICE;
    // Plain synchronise + 4-byte copy from the array's resolved address: nothing is allocated.
    cudaError_t ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) return fail(B200_ECUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(ce));
    ce = cudaMemcpy(code, dev->status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return fail(B200_ECUDA, "reading the scratch block's status word: %s", cudaGetErrorString(ce));
    return B200_OK;
}

}  // extern "C"
