// Attention forward, layouts "r2" and "r3": warp-specialised load, MMA, softmax and correction
// warpgroups in a persistent CTA (TPR = 2 or 1 softmax threads per query row).
//
// Same arithmetic as the reference kernel flash_atten_v3_fwd
// (flashattention/v3_mMnNkN/flashatten_v3.hpp:390-534): scores scaled by scale*log2(e) and
// exponentiated with exp2 against a running row max (:231-254), row sums from the un-rounded
// fp32 P, P rounded to fp16 for the P V product, final 1/sum with a zero guard, causal rule
// "row < col is masked" (:101-103); persistent tile loop as its get_tile_coord (:380-388).
//
//   warp 0  (1 thread)   TMA: per unit the two Q tiles, then K_0, V_0, K_1, V_1, ... into a ring
//   warp 1  (elected     tcgen05.mma: S_i = Q_i K_j^T and O_i += P_i V_j for both query tiles
//            lane)       of the unit, tile 1's MMAs running while tile 0's softmax runs
//   warps 4-7            correction warpgroup, one thread per query row: follows the row maxima
//                        the softmax warps publish, multiplies O_i in tensor memory by
//                        2^(old max - new max) when a max grew by more than 2^kRescaleLog2, and
//                        at the end of a unit turns O_i / sum into fp16, stages it in shared
//                        memory and stores it with TMA while the softmax warps already work on
//                        the next unit
//   warps 8-15, 16-23    TPR = 2: softmax of query tile 0 and 1, eight warps per tile, two
//                        threads per row: a thread reads one half (64 keys) of its row of S
//                        from tensor memory exactly once (tensor-memory reads are the scarce
//                        resource: a warp gets ~48 bytes per clock), the two halves exchange
//                        their maxima through shared memory, then exp2 / row sum / fp16 P
//                        written back over S, handed to the MMA warp in two parts
//   warps 8-11, 12-15    TPR = 1: four warps per tile, one thread per row holding all 128
//                        scores; the row max goes to shared memory only for the row's
//                        correction thread
//
// The MMA warp has one wait per hand-off: the first part of P_i is complete when the tile's
// softmax warps AND its correction warps have arrived (the latter meaning "O_i is rescaled, or,
// on a unit's first block, read out: it may be accumulated into").
//
// One unit = 256 query rows of one (batch, head).  CTAs walk the unit list with a static
// stride; for causal problems the grid size is chosen coprime to the number of units per head
// so every CTA sees every weight class.
//
// Tensor-memory columns: S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [256+D,256+2D); P_i
// (fp16 pairs) occupies the first 64 columns of S_i.
#pragma once

#include "fa_common.cuh"

namespace b200 {
namespace {

// TPR = softmax threads per query row.  2 (layout "r2"): 24 warps, a thread holds 64 scores.
// 1 (layout "r3"): 16 warps, a thread holds its whole row of 128 scores, no exchange of maxima.
constexpr int ws_threads(int tpr) { return 32 * (8 + 8 * tpr); }   // 2 + 2 idle, 4 correction, 8*TPR softmax
// setmaxnreg budgets.  A CTA of 768 (512) threads is launched with 80 (128) registers per
// thread, the largest multiple of 8 that fits 64 K registers; the three budgets re-divide that pool.
template <int TPR, int D>
struct WsBudget {
    static constexpr int kThreads = 32 * (8 + 8 * TPR);
    static constexpr int kRegsAtLaunch = TPR == 2 ? 80 : 128;
    // TPR = 1, measured (B4 H32 S4096 D128 / B16 H32 S2048 D64, TFLOP/s): 56/48/200 1018-1056 / 686-695,
    // 80/40/192 1050-1102 / 611 -- at head_dim 128 the MMA warp spills below ~80 registers (its
    // instruction stream is the serial resource of the loop), at 64 the larger budget only costs
    static constexpr int kRegsLoadMma = TPR == 2 ? 56 : (D == 128 ? 80 : 56);   // warps 0-3
    static constexpr int kRegsCorrection = TPR == 2 ? 40 : (D == 128 ? 40 : 48);   // warps 4-7
    static constexpr int kRegsSoftmax = TPR == 2 ? 96 : (D == 128 ? 192 : 200);    // warps 8-: 64 or 128 scores live at once
    static_assert(kRegsLoadMma * 128 + kRegsCorrection * 128 + kRegsSoftmax * 256 * TPR <= kRegsAtLaunch * kThreads,
                  "setmaxnreg budgets exceed the registers the CTA is launched with");
};
constexpr int kSmemLimit = 232448;        // 227 KiB
// P of a block is handed to the MMA warp in two parts: the first after kPart0Steps 16-key steps
// of either half of the row, the second at the end.
#ifndef B200_FA_PART0_STEPS
#define B200_FA_PART0_STEPS 2
#endif
constexpr int kPart0Steps = B200_FA_PART0_STEPS;
static_assert(kPart0Steps >= 1 && kPart0Steps <= 3, "the first part is 16, 32 or 48 keys of each half");

template <int D, int STAGES>
struct FaWsTraits {
    static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
    static constexpr int kBoxes = D / 64;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a Q tile, a K block or a V block
    static constexpr int kNumBarriers = 2 + 2 * STAGES + 2 + 4 + 8 + 2 + 2 + 2;
    // row maxima [2 block parities][2 tiles][2 halves][128] and row sums [2 tiles][2 halves][128], fp32
    static constexpr int kSmallBytes = 2 * 2 * 2 * kTileQ * 4 + 2 * 2 * kTileQ * 4 + kNumBarriers * 8 + 16;
    // tiles first (they need 1024-byte alignment for the 128-byte swizzle): Q, ring, one staging box
    static constexpr int kSmemBytes = (kQTiles + STAGES) * kTileBytes + kBoxBytes + kSmallBytes + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0;
    static constexpr int kColO = 256;
    static_assert(kSmemBytes <= kSmemLimit, "exceeds the 227 KiB shared-memory limit of sm_100");
};

__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// The running max a row's accumulators are scaled to moves only when the new maximum exceeds it
// by more than 2^kRescaleLog2 (always on the first block).  Softmax and correction threads run
// this same function on the same inputs, so they agree bit for bit.  Returns the factor
// 2^((old - new) * scale) for what was accumulated so far (1 when the reference stays).
__device__ __forceinline__ float advance_row_max(float& m, float block_max, float scale_log2) {
    const float mn = fmaxf(m, block_max);
    const bool need = (mn - m) * scale_log2 > kRescaleLog2 || m == -INFINITY;
    if (!need) return 1.f;
    const float alpha = (m == -INFINITY) ? 0.f : fast_exp2((m - mn) * scale_log2);
    m = mn;
    return alpha;
}

// P = exp2(s * scale - m * scale) for 16 scores of one row: adds the un-rounded values to the
// row sum and packs fp16 pairs (packed column x holds keys 2x, 2x+1).  EMU of every 4 pairs
// use the polynomial, the rest the SFU.
template <int EMU>
__device__ __forceinline__ void exp_16(const uint32_t* s, uint32_t (&pr)[8], f32x2 scale2, f32x2 nm2, f32x2& l,
                                       const Exp2PolyConsts& poly) {
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        const f32x2 xs = fma2(pack2(__uint_as_float(s[2 * x]), __uint_as_float(s[2 * x + 1])), scale2, nm2);
        f32x2 pp;
        if ((x & 3) < EMU) {
            pp = exp2_poly2(xs, poly);
        } else {
            float x0, x1;
            unpack2(xs, x0, x1);
            pp = pack2(fast_exp2(x0), fast_exp2(x1));
        }
        l = add2(l, pp);
        float p0, p1;
        unpack2(pp, p0, p1);
        pr[x] = pack_f16x2(p0, p1);
    }
}


template <int D, int STAGES, int EMU, int TPR>
__global__ void __launch_bounds__(WsBudget<TPR, D>::kThreads, 1)
fa_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ OMapSet tmap_o, int n_dst,
                 int seq_q, int seq_k, int heads, int q_pairs, int num_units, float scale_log2, int causal,
                 uint32_t* status) {
    using T = FaWsTraits<D, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;                                  // [2] query tiles
    const uint32_t ring_smem = q_smem + kQTiles * T::kTileBytes;        // [STAGES] K / V blocks
    const uint32_t o_smem = ring_smem + STAGES * T::kTileBytes;         // one 128 x 64 box: staging for the O stores
    const uint32_t max_smem = o_smem + kBoxBytes;                       // [2][2][TPR][128] fp32 row maxima of a block
    constexpr int kRowSlots = TPR * kTileQ;                             // one fp32 per softmax thread of a tile
    const uint32_t sum_smem = max_smem + 2 * 2 * kRowSlots * 4;         // [2][TPR][128] fp32 row sums of a finished unit
    const uint32_t bar_base = sum_smem + 2 * kRowSlots * 4;
    const uint32_t q_full = bar_base;                     // TMA -> MMA: the unit's Q tiles landed
    const uint32_t q_empty = q_full + 8;                  // MMA -> TMA: last S of the unit issued and complete
    const uint32_t kv_full = q_empty + 8;                 // [STAGES] TMA -> MMA
    const uint32_t kv_empty = kv_full + 8 * STAGES;       // [STAGES] MMA -> TMA
    const uint32_t s_full = kv_empty + 8 * STAGES;        // [2] MMA -> softmax: S_i ready
    const uint32_t p_full = s_full + 16;                  // [2][2] softmax -> MMA: part h of P_i written; the first part
                                                          // also counts the correction warps: O_i may be accumulated into
    const uint32_t max_full = p_full + 32;                // [2][4] softmax -> softmax, correction: the block's row maxima of
                                                          // one tile and lane quadrant published (the two warps that share rows)
    const uint32_t o_final = max_full + 64;               // [2] MMA -> correction: O_i of the unit complete
    const uint32_t sum_full = o_final + 16;               // [2] softmax -> correction: row sums published
    const uint32_t sum_empty = sum_full + 16;             // [2] correction -> softmax: row sums taken
    const uint32_t tmem_slot = sum_empty + 16;
    const uint32_t abort_slot = tmem_slot + 4;
    const WaitGuardS guard{abort_slot, status};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(kv_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + 8 * i, 1);
            // one arrival per softmax warp of the tile; the first part also takes one per correction
            // warp ("O_i may be accumulated into"), so the MMA warp has one wait for both
            mbar_init(p_full + 16 * i, 4 * TPR + 4);
            mbar_init(p_full + 16 * i + 8, 4 * TPR);
            for (int q = 0; q < 4; ++q) mbar_init(max_full + 32 * i + 8 * q, TPR);   // the warps that share the quadrant's rows
            mbar_init(o_final + 8 * i, 1);
            mbar_init(sum_full + 8 * i, 4 * TPR);
            mbar_init(sum_empty + 8 * i, 4);
        }
        st_shared_u32(abort_slot, 0);
        fence_mbar_init();
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        for (int d = 0; d < n_dst; ++d) prefetch_tensormap(&tmap_o.m[d]);
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, T::kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ld_shared_u32(tmem_slot);
    const int first_unit = static_cast<int>(blockIdx.x);
    const int unit_stride = static_cast<int>(gridDim.x);

    if (warp < 4) {
        setmaxnreg_dec<WsBudget<TPR, D>::kRegsLoadMma>();
        if (warp == 0 && lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            int s = 0;
            uint32_t ph = 0;
            uint32_t q_ph = 0;
            bool ok = true;
            for (int id = first_unit; id < num_units && ok; id += unit_stride) {
                const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
                ok = mbar_wait(guard, q_empty, q_ph ^ 1u, 0x1400u);
                if (!ok) break;
                q_ph ^= 1u;
                uint32_t q_bytes = 0;
                for (int i = 0; i < 2; ++i) if (u.nblk[i] > 0) q_bytes += T::kTileBytes;
                mbar_arrive_expect_tx(q_full, q_bytes);
                for (int i = 0; i < 2; ++i) {
                    if (u.nblk[i] == 0) continue;
                    for (int b = 0; b < T::kBoxes; ++b) {
                        tma_load_4d(q_smem + i * T::kTileBytes + b * kBoxBytes, &tmap_q, q_full, b * 64,
                                    u.q0 + i * kTileQ, u.head, u.batch);
                    }
                }
                for (int e = 0; e < 2 * u.nmax && ok; ++e) {  // ring entries: K_0, V_0, K_1, V_1, ...
                    ok = mbar_wait(guard, kv_empty + 8 * s, ph ^ 1u, 0x1410u + s);
                    if (!ok) break;
                    mbar_arrive_expect_tx(kv_full + 8 * s, T::kTileBytes);
                    const CUtensorMap* tm = (e & 1) ? &tmap_v : &tmap_k;
                    const int row = (e >> 1) * kTileKV;
                    for (int b = 0; b < T::kBoxes; ++b) {
                        tma_load_4d(ring_smem + s * T::kTileBytes + b * kBoxBytes, tm, kv_full + 8 * s, b * 64,
                                    row, u.head, u.batch);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer
            // The whole warp walks this code so that addresses and descriptors stay warp-uniform;
            // one elected lane issues the instructions.
            constexpr uint32_t idesc_qk = make_idesc_f16(kTileQ, kTileKV, /*fp16*/ 0, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(kTileQ, D, /*fp16*/ 0, 0, /*V is MN-major*/ 1);
            int s = 0;           // ring slot of the next entry to consume
            uint32_t ph = 0;
            uint32_t q_ph = 0;
            uint32_t p_ph[2] = {0, 0};
            bool ok = true;

            // Descriptors are built once per operand tile; a 16-element step along the head
            // dimension (S) or 16 key rows (P V) is a constant added to the address field, so one
            // MMA costs two 64-bit adds beside the instruction itself (the issuing warp shares
            // its scheduler with four softmax warps).
            const uint64_t q_desc0 = smem_desc_kmajor_sw128(q_smem);
            const uint64_t q_desc1 = smem_desc_kmajor_sw128(q_smem + T::kTileBytes);
            auto issue_s = [&](int i, uint32_t k_addr) {
                const uint64_t q_desc = i ? q_desc1 : q_desc0;
                const uint64_t k_desc = smem_desc_kmajor_sw128(k_addr);
                if (!elect_one()) return;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    constexpr int kBoxUnits = kBoxBytes >> 4;
                    const uint64_t off = static_cast<uint64_t>((kk >> 2) * kBoxUnits + (kk & 3) * 2);
                    mma_ss<1>(tmem_base + T::kColS + i * kTileKV, q_desc + off, k_desc + off, idesc_qk,
                              kk > 0 ? 1u : 0u);
                }
            };
            // Part h of P V.  The two threads of a row work on keys [0,64) and [64,128) at the
            // same time, so the first part is the first kPart0Steps 16-key steps of either half
            // (steps 0.. of keys [0,64) and steps 4.. of keys [64,128)), the second part the
            // rest.  P: 16 keys = 8 packed columns.  V: 16 key rows = 2048 bytes; the second
            // 64-wide span of the head dimension lives one box (16 KiB) further.
            auto issue_pv_part = [&](int i, int h, uint64_t v_desc, bool accumulate) {
                if (!elect_one()) return;
                bool first = !accumulate;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const bool in_part0 = (TPR == 2) ? ((kk & 3) < kPart0Steps) : (kk < kPart0Steps);
                    if (in_part0 != (h == 0)) continue;
                    mma_ts(tmem_base + T::kColO + i * D, tmem_base + T::kColS + i * kTileKV + kk * 8,
                           v_desc + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv, first ? 0u : 1u);
                    first = false;
                }
            };
            auto commit = [&](uint32_t bar) {
                if (elect_one()) mma_commit<1>(bar);
            };
            // every lane polls; the outcome is made warp-uniform so the elections stay convergent
            auto wait = [&](uint32_t bar, uint32_t parity, uint32_t site) {
                return __all_sync(0xffffffffu, mbar_wait(guard, bar, parity, site));
            };

            FA_PROF_DECL
            for (int id = first_unit; id < num_units && ok; id += unit_stride) {
                const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
                FA_PROF(5)
                ok = wait(q_full, q_ph, 0x1200u);
                if (!ok) break;
                FA_PROF(0)
                q_ph ^= 1u;
                // K_0
                uint32_t k_addr = 0;
                uint64_t v_desc = 0;
                int k_slot = 0, v_slot = 0;
                ok = wait(kv_full + 8 * s, ph, 0x1210u + s);
                if (!ok) break;
                FA_PROF(1)
                k_addr = ring_smem + s * T::kTileBytes;
                k_slot = s;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                tc_fence_after();
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (u.nblk[i] > 0) {
                        issue_s(i, k_addr);
                        commit(s_full + 8 * i);
                    }
                }
                commit(kv_empty + 8 * k_slot);
                if (u.nmax == 1) commit(q_empty);
                for (int j = 0; j < u.nmax && ok; ++j) {
                    // V_j
                    FA_PROF(5)
                    ok = wait(kv_full + 8 * s, ph, 0x1220u + s);
                    if (!ok) break;
                    FA_PROF(1)
                    v_desc = smem_desc_mnmajor_sw128(ring_smem + s * T::kTileBytes, kBoxBytes);
                    v_slot = s;
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                    bool have_k = false;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        if (!ok || j >= u.nblk[i]) continue;
                        FA_PROF(5)
                        ok = wait(p_full + 16 * i, p_ph[i], 0x1230u + i);
                        if (!ok) continue;
                        FA_PROF(3 + i)
                        tc_fence_after();
                        issue_pv_part(i, 0, v_desc, j > 0);
                        FA_PROF(5)
                        ok = wait(p_full + 16 * i + 8, p_ph[i], 0x1238u + i);
                        if (!ok) continue;
                        FA_PROF(6 + i)
                        p_ph[i] ^= 1u;
                        tc_fence_after();
                        issue_pv_part(i, 1, v_desc, true);
                        if (j + 1 < u.nblk[i]) {
                            if (!have_k) {
                                FA_PROF(5)
                                ok = wait(kv_full + 8 * s, ph, 0x1240u + s);
                                if (!ok) continue;
                                FA_PROF(1)
                                tc_fence_after();
                                k_addr = ring_smem + s * T::kTileBytes;
                                k_slot = s;
                                if (++s == STAGES) { s = 0; ph ^= 1u; }
                                have_k = true;
                            }
                            issue_s(i, k_addr);
                            commit(s_full + 8 * i);
                        } else {
                            commit(o_final + 8 * i);
                        }
                    }
                    if (!ok) break;
                    commit(kv_empty + 8 * v_slot);
                    if (j + 1 < u.nmax) {
                        // the tile with nmax blocks took K_{j+1} above
                        commit(kv_empty + 8 * k_slot);
                        if (j + 2 == u.nmax) commit(q_empty);   // that was the unit's last S
                    }
                }
            }
            FA_PROF(5)
            FA_PROF_DUMP(0)
        }
    } else if (warp < 8) {
        setmaxnreg_dec<WsBudget<TPR, D>::kRegsCorrection>();
        // --------------------------------------------------------------- correction warpgroup
        const int quad = warp & 3;                      // tensor-memory lane quadrant
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        uint32_t x_ph[2] = {0, 0};                      // max_full: one completion per block of the tile
        uint32_t u_ph[2] = {0, 0};                      // sum_full / o_final: one completion per unit the tile takes part in
        float m_run[2] = {-INFINITY, -INFINITY};        // the same running max the row's softmax threads keep
        bool ok = true;
        FA_PROF_DECL
        // One block of tile i: take the row maxima the softmax threads published, advance the
        // running max, rescale O_i if it moved, and tell the MMA warp that O_i may be accumulated
        // into.  Every block is acknowledged, the first of a unit included (there the arrival
        // also says that the previous unit's epilogue has read O_i): the softmax warps can then
        // never get two blocks ahead of this warp, which a one-bit barrier phase could not tell
        // from none.
        auto handle_block = [&](int i, bool first) {
            FA_PROF(1)
            ok = __all_sync(0xffffffffu, mbar_wait(guard, max_full + 32 * i + 8 * quad, x_ph[i] & 1u, 0x1500u + i));
            if (!ok) return;
            FA_PROF(0)
            const uint32_t box = max_smem + (((x_ph[i] & 1u) * 2 + i) * kRowSlots + row_in_tile) * 4;
            ++x_ph[i];
            const float block_max = (TPR == 2) ? fmaxf(ld_shared_f32(box), ld_shared_f32(box + kTileQ * 4)) : ld_shared_f32(box);
            if (first) m_run[i] = -INFINITY;
            const float alpha = advance_row_max(m_run[i], block_max, scale_log2);
            if (!first && __any_sync(0xffffffffu, alpha != 1.f)) {
                tc_fence_after();
                const uint32_t t_o = tmem_base + lane_base + T::kColO + i * D;
#pragma unroll 1
                for (int c = 0; c < D / 16; ++c) {
                    uint32_t o[16];
                    tmem_ld_32x32b_x16(t_o + c * 16, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 16; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
                    tmem_st_32x32b_x16(t_o + c * 16, o);
                }
                tmem_wait_st();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 16 * i);
        };
        if (first_unit < num_units) {
            const UnitCoord u0 = unit_coord(first_unit, q_pairs, heads, seq_q, seq_k, causal);
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (ok && u0.nblk[i] > 0) handle_block(i, true);
        }
        for (int id = first_unit; id < num_units && ok; id += unit_stride) {
            const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
            // which tiles the CTA's next unit uses (its first block is acknowledged right after
            // this unit's epilogue of the same tile)
            bool next_has[2] = {false, false};
            if (id + unit_stride < num_units) {
                const UnitCoord un = unit_coord(id + unit_stride, q_pairs, heads, seq_q, seq_k, causal);
                next_has[0] = un.nblk[0] > 0;
                next_has[1] = un.nblk[1] > 0;
            }
            for (int j = 1; j < u.nmax && ok; ++j) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (!ok || j >= u.nblk[i]) continue;
                    handle_block(i, false);
                }
            }
            // ---------------------------------------------------------------------- epilogue
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (!ok || u.nblk[i] == 0) continue;
                FA_PROF(1)
                ok = __all_sync(0xffffffffu, mbar_wait(guard, sum_full + 8 * i, u_ph[i], 0x1510u + i));
                if (!ok) continue;
                const uint32_t sums = sum_smem + (i * kRowSlots + row_in_tile) * 4;
                const float l = (TPR == 2) ? ld_shared_f32(sums) + ld_shared_f32(sums + kTileQ * 4) : ld_shared_f32(sums);
                __syncwarp();
                if (lane == 0) mbar_arrive(sum_empty + 8 * i);
                ok = __all_sync(0xffffffffu, mbar_wait(guard, o_final + 8 * i, u_ph[i], 0x1518u + i));
                if (!ok) continue;
                FA_PROF(2)
                tc_fence_after();
                const float inv = (l == 0.f) ? 1.f : (1.f / l);
                const uint32_t t_o = tmem_base + lane_base + T::kColO + i * D;
                const uint32_t row_addr = o_smem + row_in_tile * 128;
#pragma unroll 1
                for (int c = 0; c < D / 16; ++c) {
                    uint32_t o[16];
                    tmem_ld_32x32b_x16(t_o + c * 16, o);
                    tmem_wait_ld();
                    if ((c & 3) == 0) {
                        // a new 64-column box: the stores issued so far have read this warp's staging rows
                        if (lane == 0) tma_store_wait_read<0>();
                        __syncwarp();
                    }
                    uint32_t h[8];
#pragma unroll
                    for (int x = 0; x < 8; ++x)
                        h[x] = pack_f16x2(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
                    const int chunk = (c & 3) * 2;       // 16-byte chunks of the 128-byte staging row
                    st_shared_v4(row_addr + ((chunk ^ (row_in_tile & 7)) << 4), h[0], h[1], h[2], h[3]);
                    st_shared_v4(row_addr + (((chunk + 1) ^ (row_in_tile & 7)) << 4), h[4], h[5], h[6], h[7]);
                    if ((c & 3) == 3) {
                        // the box is complete: this warp's 32 rows of it, to every destination
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            for (int d = 0; d < n_dst; ++d)
                                tma_store_4d(&tmap_o.m[d], o_smem + quad * 32 * 128, (c >> 2) * 64,
                                             u.q0 + i * kTileQ + quad * 32, u.head, u.batch);
                            tma_store_commit();
                        }
                    }
                }
                u_ph[i] ^= 1u;
                FA_PROF(3)
                // O_i has been read: first block of the CTA's next unit, if this tile has one
                if (next_has[i]) handle_block(i, true);
            }
        }
        if (lane == 0) tma_store_wait_read<0>();   // shared memory may go; the writes finish on their own before the grid does
        if (warp == 4) FA_PROF_DUMP(24)
    } else {
        setmaxnreg_inc<WsBudget<TPR, D>::kRegsSoftmax>();
        // ------------------------------------------------------------------ softmax warps
        const int i = (warp - 8) / (4 * TPR);           // query tile of this warp
        const int quad = warp & 3;                      // tensor-memory lane quadrant
        const int half = (TPR == 2) ? ((warp - 8) >> 2) & 1 : 0;   // which 64 keys of the block (two threads per row)
        const int row_in_tile = quad * 32 + lane;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + T::kColS + i * kTileKV;
        const uint32_t t_s = t_row + half * 64;         // this thread's scores
        const uint32_t t_p = t_row + half * 32;         // where its P goes (packed pairs)
        const Exp2PolyConsts poly = make_exp2_poly_consts();
        const f32x2 scale2 = pack2(scale_log2, scale_log2);
        uint32_t blocks_done = 0;                       // parity of s_full / max_full and of the maxima slot
        uint32_t units_done = 0;
        bool ok = true;
        FA_PROF_DECL
        for (int id = first_unit; id < num_units && ok; id += unit_stride) {
            const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
            const int n = i ? u.nblk[1] : u.nblk[0];
            if (n == 0) continue;
            const int grow = u.q0 + i * kTileQ + row_in_tile;   // query index of this row in the sequence
            float m = -INFINITY;                        // running max the accumulators are scaled to
            f32x2 l = pack2(0.f, 0.f);                  // partial row sum (this thread's keys)
            for (int j = 0; j < n && ok; ++j) {
                FA_PROF(4)
                const uint32_t par = blocks_done & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(guard, s_full + 8 * i, par, 0x1300u + i));
                if (!ok) break;
                FA_PROF(0)
                tc_fence_after();
                if constexpr (TPR == 1) {
                    // one thread per row: the whole row of 128 scores, no partner
                    uint32_t sr[4][32];
                    tmem_ld_32x32b_x32(t_row + 0, sr[0]);
                    tmem_ld_32x32b_x32(t_row + 32, sr[1]);
                    tmem_ld_32x32b_x32(t_row + 64, sr[2]);
                    tmem_ld_32x32b_x32(t_row + 96, sr[3]);
                    tmem_wait_ld();
                    const int col0 = j * kTileKV;
                    if ((col0 + kTileKV > seq_k) || (causal && (col0 + kTileKV - 1 > u.q0 + i * kTileQ))) {
                        const int limit = causal ? min(seq_k - 1, grow) : (seq_k - 1);  // last visible key
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int x = 0; x < 32; ++x)
                                if (col0 + c * 32 + x > limit) sr[c][x] = 0xff800000u;  // -inf
                    }
                    float mc[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        mc[c] = max3(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
#pragma unroll
                        for (int x = 3; x < 31; x += 2)
                            mc[c] = max3(mc[c], __uint_as_float(sr[c][x]), __uint_as_float(sr[c][x + 1]));
                        mc[c] = fmaxf(mc[c], __uint_as_float(sr[c][31]));
                    }
                    const float block_max = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
                    // for the row's correction thread
                    st_shared_f32(max_smem + ((par * 2 + i) * kRowSlots + row_in_tile) * 4, block_max);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(max_full + 32 * i + 8 * quad);
                    const float alpha = advance_row_max(m, block_max, scale_log2);
                    l = mul2(l, pack2(alpha, alpha));
                    ++blocks_done;
                    FA_PROF(1)
                    const float nm = -((m == -INFINITY) ? 0.f : m) * scale_log2;
                    const f32x2 nm2 = pack2(nm, nm);
                    uint32_t pr[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        exp_16<EMU>(&sr[c >> 1][(c & 1) * 16], pr, scale2, nm2, l, poly);
                        tmem_st_32x32b_x8(t_row + 8 * c, pr);    // 16 keys -> 8 packed columns
                        if (c == kPart0Steps - 1 || c == 7) {
                            tmem_wait_st();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(p_full + 16 * i + (c == 7 ? 8 : 0));
                            if (c != 7) FA_PROF(2)
                        }
                    }
                    FA_PROF(3)
                    continue;
                }
                uint32_t sa[32], sb[32];
                tmem_ld_32x32b_x32(t_s, sa);
                tmem_ld_32x32b_x32(t_s + 32, sb);
                tmem_wait_ld();
                const int col0 = j * kTileKV + half * 64;
                if ((col0 + 64 > seq_k) || (causal && (col0 + 63 > u.q0 + i * kTileQ))) {
                    const int limit = causal ? min(seq_k - 1, grow) : (seq_k - 1);  // last visible key
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        if (col0 + x > limit) sa[x] = 0xff800000u;  // -inf
                        if (col0 + 32 + x > limit) sb[x] = 0xff800000u;
                    }
                }
                // four independent chains
                float mc[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t* s = (c < 2 ? sa : sb) + (c & 1) * 16;
                    mc[c] = max3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
#pragma unroll
                    for (int x = 3; x < 15; x += 2) mc[c] = max3(mc[c], __uint_as_float(s[x]), __uint_as_float(s[x + 1]));
                    mc[c] = fmaxf(mc[c], __uint_as_float(s[15]));
                }
                const float mine = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
                // exchange with the thread that holds the other 64 keys of this row
                const uint32_t box = max_smem + ((par * 2 + i) * kRowSlots + row_in_tile) * 4;
                st_shared_f32(box + half * kTileQ * 4, mine);
                __syncwarp();
                if (lane == 0) mbar_arrive(max_full + 32 * i + 8 * quad);
                ok = __all_sync(0xffffffffu, mbar_wait(guard, max_full + 32 * i + 8 * quad, par, 0x1308u + i));
                if (!ok) break;
                const float theirs = ld_shared_f32(box + (half ^ 1) * kTileQ * 4);
                // fmaxf in the order the correction thread uses (half 0, half 1)
                const float block_max = half ? fmaxf(theirs, mine) : fmaxf(mine, theirs);
                const float alpha = advance_row_max(m, block_max, scale_log2);
                l = mul2(l, pack2(alpha, alpha));
                ++blocks_done;
                FA_PROF(1)
                const float nm = -((m == -INFINITY) ? 0.f : m) * scale_log2;
                const f32x2 nm2 = pack2(nm, nm);
                uint32_t pr[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    exp_16<EMU>((c < 2 ? sa : sb) + (c & 1) * 16, pr, scale2, nm2, l, poly);
                    tmem_st_32x32b_x8(t_p + 8 * c, pr);      // 16 keys of this half -> 8 packed columns
                    if (c == kPart0Steps - 1 || c == 3) {
                        tmem_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(p_full + 16 * i + (c == 3 ? 8 : 0));
                        if (c != 3) FA_PROF(2)
                    }
                }
                FA_PROF(3)
            }
            if (!ok) break;
            // ------------------------------------------------ row sums of the finished unit
            float t0, t1;
            unpack2(l, t0, t1);
            if (units_done > 0) {
                // the correction warps have taken the previous unit's sums
                ok = __all_sync(0xffffffffu, mbar_wait(guard, sum_empty + 8 * i, (units_done - 1) & 1u, 0x1310u + i));
                if (!ok) break;
            }
            st_shared_f32(sum_smem + (i * kRowSlots + half * kTileQ + row_in_tile) * 4, t0 + t1);
            __syncwarp();
            if (lane == 0) mbar_arrive(sum_full + 8 * i);
            ++units_done;
        }
        if (warp == 8) FA_PROF_DUMP(8)
        if (warp == 8 + 4 * TPR) FA_PROF_DUMP(16)
    }

    // --------------------------------------------------------------------------- teardown
    if (ld_shared_u32(abort_slot) != 0) {
        for (int it = 0; it < 64; ++it) __nanosleep(100000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc<1>(tmem_base, T::kTmemCols);
    }
}

}  // namespace
}  // namespace b200
