// Attention forward, layout "r4": the row-thread kernel (layout r1: one softmax thread per
// query row that also rescales O) made persistent.  A CTA walks units of 256 query rows with a
// static stride, so barriers, tensor memory and tensor-map prefetches are set up once, and the
// next unit's Q, K_0, V_0, ... are already in flight (and its first S = Q K^T issued) while the
// softmax warps write the current unit's output.
//
//   warp 0  (1 thread)  TMA: per unit the two Q tiles (as soon as the previous unit's last S has
//                       been issued and completed), then K_0, V_0, K_1, V_1, ... into the ring
//   warp 1  (elected    tcgen05.mma: S_i = Q_i K_j^T and O_i += P_i V_j for both query tiles of
//            lane)      the unit, tile 1's MMAs running while tile 0's softmax runs
//   warps 4-7, 8-11     one softmax warpgroup per query tile, one thread per row: reads S_i
//                       from tensor memory, running max / sum in registers, writes P_i (fp16)
//                       over S_i, rescales O_i in tensor memory only when the row max grew by
//                       more than 2^kRescaleLog2; at the end of a unit O_i / sum -> fp16 ->
//                       a staging box of its own (not the Q tile: that is being reloaded) ->
//                       TMA store, 64 columns at a time
//
// Same arithmetic as layout r1 (fa_fwd_rowthread.cuh) and as the reference kernel
// flash_atten_v3_fwd (flashattention/v3_mMnNkN/flashatten_v3.hpp:390-534); persistent tile
// loop as its get_tile_coord (:380-388).
//
// Tensor-memory columns: S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [256+D,256+2D).
#pragma once

#include "fa_common.cuh"
#include "fa_fwd_rowthread.cuh"   // kFaThreads, kSplitP, register budgets

namespace b200 {
namespace {

// setmaxnreg budgets out of the 168 x 384 registers the CTA is launched with.  The unit loop
// keeps a few more values live in every role than layout r1 does; these splits leave at most
// 16 bytes of spills (r1's 56 / 224 would spill ~100 here).
template <int D>
struct FaPersBudget {
    static constexpr int kRegsLoadMma = D == 128 ? 80 : 72;      // warps 0-3
    static constexpr int kRegsSoftmax = D == 128 ? 208 : 216;    // warps 4-11
    static_assert(kRegsLoadMma * 128 + kRegsSoftmax * 256 <= kRegsAtLaunch * kFaThreads,
                  "setmaxnreg budgets exceed the registers the CTA is launched with");
};

template <int D, int STAGES>
struct FaPersTraits {
    static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
    static constexpr int kBoxes = D / 64;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a Q tile, a K block or a V block
    static constexpr int kNumBarriers = 2 + 2 * STAGES + 2 + 4 + 2;
    // Q tiles, ring, one 128 x 64 staging box per query tile
    static constexpr int kSmemBytes = (kQTiles + STAGES) * kTileBytes + kQTiles * kBoxBytes + kNumBarriers * 8 + 16 + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0;
    static constexpr int kColO = 256;
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB shared-memory limit of sm_100");
};

template <int D, int STAGES, int EMU>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd_pers_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ OMapSet tmap_o, int n_dst,
                   int seq_q, int seq_k, int heads, int q_pairs, int num_units, float scale_log2, int causal,
                   uint32_t* status) {
    using T = FaPersTraits<D, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;                               // [2] query tiles
    const uint32_t ring_smem = smem_base + kQTiles * T::kTileBytes;  // [STAGES] K / V blocks
    const uint32_t o_smem = ring_smem + STAGES * T::kTileBytes;      // [2] 128 x 64 staging boxes for the O stores
    const uint32_t bar_base = o_smem + kQTiles * kBoxBytes;
    const uint32_t q_full = bar_base;                     // TMA -> MMA: the unit's Q tiles landed
    const uint32_t q_empty = q_full + 8;                  // MMA -> TMA: the unit's last S issued and complete
    const uint32_t kv_full = q_empty + 8;                 // [STAGES] TMA -> MMA
    const uint32_t kv_empty = kv_full + 8 * STAGES;       // [STAGES] MMA -> TMA
    const uint32_t s_full = kv_empty + 8 * STAGES;        // [2] MMA -> softmax: S_i ready
    const uint32_t p_full = s_full + 16;                  // [2][2] softmax -> MMA: part h of P_i written (and O_i rescaled)
    // [2] MMA -> softmax: O_i of the unit complete.  A barrier of its own: the next unit's first
    // S_i is issued while the softmax warps are still in this unit's epilogue, and two
    // completions of one barrier ahead of its waiter cannot be told from none (one-bit phase).
    const uint32_t o_final = p_full + 32;
    const uint32_t tmem_slot = o_final + 16;
    const uint32_t abort_slot = tmem_slot + 4;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
    volatile uint32_t* abort_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));
    const WaitGuard guard{abort_ptr, status};

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
            mbar_init(o_final + 8 * i, 1);
            mbar_init(p_full + 16 * i, 4);      // one arrival per softmax warp
            mbar_init(p_full + 16 * i + 8, 4);
        }
        *abort_ptr = 0;
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
    const uint32_t tmem_base = *tmem_slot_ptr;
    const int first_unit = static_cast<int>(blockIdx.x);
    const int unit_stride = static_cast<int>(gridDim.x);

    if (warp < 4) {
        setmaxnreg_dec<FaPersBudget<D>::kRegsLoadMma>();
        if (warp == 0 && lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            int s = 0;
            uint32_t ph = 0;
            uint32_t q_ph = 0;
            bool ok = true;
            for (int slot = first_unit; ok; slot += unit_stride) {
                const int id = schedule_unit(slot, first_unit, unit_stride, causal);
                if (id >= num_units) break;
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
                    ok = mbar_wait(guard, kv_empty + 8 * s, ph ^ 1u, 0x1100u + s);
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
            // Part h of P V: 16-key steps [0,kSplitP) or [kSplitP,8) of the block.
            auto issue_pv_half = [&](int i, int h, uint32_t v_addr, bool accumulate) {
                const uint64_t v_desc = smem_desc_mnmajor_sw128(v_addr, kBoxBytes);
                if (!elect_one()) return;
#pragma unroll
                for (int kk = (h ? kSplitP : 0); kk < (h ? 8 : kSplitP); ++kk) {
                    mma_ts(tmem_base + T::kColO + i * D, tmem_base + T::kColS + i * kTileKV + kk * 8,
                           v_desc + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv,
                           (accumulate || kk > 0) ? 1u : 0u);
                }
            };
            auto commit = [&](uint32_t bar) {
                if (elect_one()) mma_commit<1>(bar);
            };
            // every lane polls; the outcome is made warp-uniform so the elections stay convergent
            auto wait = [&](uint32_t bar, uint32_t parity, uint32_t site) {
                return __all_sync(0xffffffffu, mbar_wait(guard, bar, parity, site));
            };

            for (int slot = first_unit; ok; slot += unit_stride) {
                const int id = schedule_unit(slot, first_unit, unit_stride, causal);
                if (id >= num_units) break;
                const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
                ok = wait(q_full, q_ph, 0x1200u);
                if (!ok) break;
                q_ph ^= 1u;
                // K_0
                uint32_t k_addr = 0, v_addr = 0;
                int k_slot = 0, v_slot = 0;
                ok = wait(kv_full + 8 * s, ph, 0x1210u + s);
                if (!ok) break;
                k_addr = ring_smem + s * T::kTileBytes;
                k_slot = s;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                tc_fence_after();
                // (S_i of the new unit overwrites P_i of the previous unit's last block: the tensor
                // pipe executes in issue order, and that block's P V was issued before)
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
                    ok = wait(kv_full + 8 * s, ph, 0x1220u + s);
                    if (!ok) break;
                    v_addr = ring_smem + s * T::kTileBytes;
                    v_slot = s;
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                    bool have_k = false;
                    for (int i = 0; i < 2 && ok; ++i) {
                        if (j >= u.nblk[i]) continue;
                        if constexpr (kSplitP > 0) {
                            ok = wait(p_full + 16 * i, p_ph[i], 0x1230u + i);
                            if (!ok) break;
                            tc_fence_after();
                            issue_pv_half(i, 0, v_addr, j > 0);
                        }
                        ok = wait(p_full + 16 * i + 8, p_ph[i], 0x1238u + i);
                        if (!ok) break;
                        p_ph[i] ^= 1u;
                        tc_fence_after();
                        issue_pv_half(i, 1, v_addr, kSplitP > 0 || j > 0);
                        if (j + 1 < u.nblk[i]) {
                            if (!have_k) {
                                ok = wait(kv_full + 8 * s, ph, 0x1240u + s);
                                if (!ok) break;
                                tc_fence_after();
                                k_addr = ring_smem + s * T::kTileBytes;
                                k_slot = s;
                                if (++s == STAGES) { s = 0; ph ^= 1u; }
                                have_k = true;
                            }
                            issue_s(i, k_addr);
                            commit(s_full + 8 * i);
                        } else {
                            commit(o_final + 8 * i);    // that was the tile's last block
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
        }
    } else {
        setmaxnreg_inc<FaPersBudget<D>::kRegsSoftmax>();
        // ------------------------------------------------------------- softmax warpgroups
        const int i = (warp - 4) >> 2;                 // query tile of this warpgroup
        const int quad = warp & 3;                     // tensor-memory lane quadrant
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_s = tmem_base + lane_base + T::kColS + i * kTileKV;
        const uint32_t t_o = tmem_base + lane_base + T::kColO + i * D;
        const uint32_t stage = o_smem + i * kBoxBytes;  // this tile's staging box
        const Exp2PolyConsts poly = make_exp2_poly_consts();
        uint32_t s_count = 0;                          // completions of s_full[i] consumed so far
        uint32_t units_done = 0;                       // completions of o_final[i] consumed so far
        bool ok = true;
        for (int slot = first_unit; ok; slot += unit_stride) {
            const int id = schedule_unit(slot, first_unit, unit_stride, causal);
            if (id >= num_units) break;
            const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
            const int n = i ? u.nblk[1] : u.nblk[0];
            if (n == 0) continue;
            const int row = u.q0 + i * kTileQ + row_in_tile;  // query index in the sequence
            float m = -INFINITY;  // running max the accumulators are scaled to
            float l0 = 0.f, l1 = 0.f;  // running sum of exp2(s*scale - m*scale), two partial sums
            for (int j = 0; j < n && ok; ++j) {
                ok = mbar_wait(guard, s_full + 8 * i, s_count & 1u, 0x1300u + i);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ++s_count;
                tc_fence_after();
                uint32_t sr[4][32];
                tmem_ld_32x32b_x32(t_s + 0, sr[0]);
                tmem_ld_32x32b_x32(t_s + 32, sr[1]);
                tmem_ld_32x32b_x32(t_s + 64, sr[2]);
                tmem_ld_32x32b_x32(t_s + 96, sr[3]);
                tmem_wait_ld();
                const int col0 = j * kTileKV;
                const bool need_mask = (col0 + kTileKV > seq_k) || (causal && (col0 + kTileKV - 1 > u.q0 + i * kTileQ));
                if (need_mask) {
                    const int limit = causal ? min(seq_k - 1, row) : (seq_k - 1);  // last visible key
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (col0 + c * 32 + x > limit) sr[c][x] = 0xff800000u;  // -inf
                }
                // Four independent chains (one per 32-column chunk) instead of one 64-deep chain.
                float mc[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    mc[c] = max3(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
#pragma unroll
                    for (int x = 3; x < 31; x += 2)
                        mc[c] = max3(mc[c], __uint_as_float(sr[c][x]), __uint_as_float(sr[c][x + 1]));
                    mc[c] = fmaxf(mc[c], __uint_as_float(sr[c][31]));
                }
                const float mblk = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
                const float m_new = fmaxf(m, mblk);
                // Rescale only when the max moved enough to matter (always on the first block).
                const bool need = (m_new - m) * scale_log2 > kRescaleLog2 || m == -INFINITY;
                if (__any_sync(0xffffffffu, need)) {
                    const float m_use = need ? m_new : m;
                    const float alpha = (m == -INFINITY) ? 0.f : fast_exp2((m - m_use) * scale_log2);
                    l0 *= alpha;
                    l1 *= alpha;
                    m = m_use;
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t o[32];
                            tmem_ld_32x32b_x32(t_o + c * 32, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
                            tmem_st_32x32b_x32(t_o + c * 32, o);
                        }
                    }
                }
                const float m_fin = (m == -INFINITY) ? 0.f : m;
                const float neg_m = -m_fin * scale_log2;
                const f32x2 scale2 = pack2(scale_log2, scale_log2);
                const f32x2 neg_m2 = pack2(neg_m, neg_m);
                f32x2 lsum[4] = {pack2(l0, l1), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pr[16];
#pragma unroll
                    for (int x = 0; x < 32; x += 2) {
                        const f32x2 xs = fma2(pack2(__uint_as_float(sr[c][x]), __uint_as_float(sr[c][x + 1])), scale2, neg_m2);
                        f32x2 pp;
                        // EMU of every 4 pairs take the polynomial path, the rest the SFU.
                        if (((x >> 1) & 3) < EMU) {
                            pp = exp2_poly2(xs, poly);
                        } else {
                            float a, b;
                            unpack2(xs, a, b);
                            pp = pack2(fast_exp2(a), fast_exp2(b));
                        }
                        lsum[c] = add2(lsum[c], pp);
                        float p0, p1;
                        unpack2(pp, p0, p1);
                        pr[x >> 1] = pack_f16x2(p0, p1);
                    }
                    // 32 keys = 16 packed columns; S is already in registers, so P may overwrite it.
                    tmem_st_32x32b_x16(t_s + c * 16, pr);
                    if ((kSplitP > 0 && c == kSplitP / 2 - 1) || c == 3) {
                        // The first part (or all) of P is in tensor memory: let the MMA warp start on it.
                        tmem_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(p_full + 16 * i + 8 * (c == 3 ? 1 : 0));
                    }
                }
                unpack2(add2(add2(lsum[0], lsum[1]), add2(lsum[2], lsum[3])), l0, l1);
            }
            if (!ok) break;
            // ---------------------------------------------------------------------- epilogue
            const float l = l0 + l1;
            ok = mbar_wait(guard, o_final + 8 * i, units_done & 1u, 0x1310u + i);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ++units_done;
            tc_fence_after();
            const float inv = (l == 0.f) ? 1.f : (1.f / l);
#pragma unroll 1
            for (int b = 0; b < T::kBoxes; ++b) {     // 64 output columns at a time through the tile's staging box
                // the previous store of this tile (previous box, or the previous unit) has read the box
                if (row_in_tile == 0) tma_store_wait_read<0>();
                named_bar_sync(1 + i, kTileQ);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32b_x32(t_o + b * 64 + c * 32, o);
                    tmem_wait_ld();
                    uint32_t h[16];
#pragma unroll
                    for (int x = 0; x < 16; ++x)
                        h[x] = pack_f16x2(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
                    const uint32_t row_addr = stage + row_in_tile * 128;
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int chunk = c * 4 + jj;
                        st_shared_v4(row_addr + ((chunk ^ (row_in_tile & 7)) << 4), h[4 * jj], h[4 * jj + 1],
                                     h[4 * jj + 2], h[4 * jj + 3]);
                    }
                }
                fence_proxy_async_smem();
                named_bar_sync(1 + i, kTileQ);
                if (row_in_tile == 0) {
                    for (int d = 0; d < n_dst; ++d)
                        tma_store_4d(&tmap_o.m[d], stage, b * 64, u.q0 + i * kTileQ, u.head, u.batch);
                    tma_store_commit();
                }
            }
            // O_i has been read out of tensor memory by every thread of this warpgroup before any
            // of them hands over the next unit's first P (program order per thread, and the
            // hand-off barrier needs all four warps), so P V of that block may overwrite O_i.
        }
        if (row_in_tile == 0) tma_store_wait_read<0>();   // shared memory may go; the writes finish on their own before the grid does
    }

    // --------------------------------------------------------------------------- teardown
    if (*abort_ptr != 0) {
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
