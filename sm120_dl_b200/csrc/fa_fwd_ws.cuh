// Attention forward, layout "r4": warp-specialised load, MMA, softmax and correction
// warpgroups in a persistent CTA.
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
//   warps 4-7            correction warpgroup, one thread per query row: multiplies O_i in
//                        tensor memory by the factor the softmax warps publish when a row max
//                        grew by more than 2^kRescaleLog2, and at the end of a unit turns
//                        O_i / sum into fp16, stages it in shared memory and stores it with
//                        TMA while the softmax warps already work on the next unit
//   warps 8-15, 16-23    softmax of query tile 0 and 1, eight warps per tile.  A warp owns 16
//                        rows; a row's 128 scores are spread over the four threads of a quad
//                        (the m16n8 fragment layout of tcgen05.ld.16x256b), so a row max costs
//                        two shuffles and a thread never holds more than 32 scores: first pass
//                        row max, second pass exp2 / row sum / fp16 P written back over S in
//                        tensor memory, handed to the MMA warp in two halves of 64 keys.
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

constexpr int kWsThreads = 768;           // 24 warps: 2 + 2 idle, 4 correction, 16 softmax
// setmaxnreg budgets.  A CTA of 768 threads is launched with 80 registers per thread (the
// largest multiple of 8 that fits 64 K registers); the three budgets re-divide exactly that pool.
constexpr int kWsRegsAtLaunch = 80;
constexpr int kWsRegsLoadMma = 56;        // warps 0-3
constexpr int kWsRegsCorrection = 72;     // warps 4-7
constexpr int kWsRegsSoftmax = 88;        // warps 8-23
static_assert(kWsRegsLoadMma * 128 + kWsRegsCorrection * 128 + kWsRegsSoftmax * 512 <= kWsRegsAtLaunch * kWsThreads,
              "setmaxnreg budgets exceed the registers the CTA is launched with");
constexpr int kSmemLimit = 232448;        // 227 KiB

template <int D, int STAGES>
struct FaWsTraits {
    static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
    static constexpr int kBoxes = D / 64;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a Q tile, a K block, a V block or an O tile
    static constexpr int kNumBarriers = 2 + 2 * STAGES + 2 + 4 + 2 + 2 + 2 + 2 + 2;
    static constexpr int kSmallBytes = 2 * kTileQ * 4 /* alpha */ + 2 * kTileQ * 4 /* totals */ + kNumBarriers * 8 + 16;
    // data that must start on a 1024-byte boundary (128-byte swizzle), then the small arrays
    static constexpr int kNeeded = (kQTiles + STAGES + 1) * kTileBytes + kSmallBytes;
    static constexpr int kSmemBytes = (kNeeded + 1024 <= kSmemLimit) ? kNeeded + 1024 : kSmemLimit;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0;
    static constexpr int kColO = 256;
    static_assert(kNeeded <= kSmemLimit, "exceeds the 227 KiB shared-memory limit of sm_100");
};

__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// (pair of the head, head, batch) of unit `id`, and the key blocks its two tiles visit.
struct UnitCoord {
    int q0, head, batch;
    int nblk[2];
    int nmax;
};
__device__ __forceinline__ UnitCoord unit_coord(int id, int q_pairs, int heads, int seq_q, int seq_k, int causal) {
    UnitCoord u;
    const int hb = id / q_pairs;
    const int p = id - hb * q_pairs;
    const int pair = causal ? (q_pairs - 1 - p) : p;   // heaviest causal units of a head first
    u.batch = hb / heads;
    u.head = hb - u.batch * heads;
    u.q0 = pair * (kQTiles * kTileQ);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row0 = u.q0 + i * kTileQ;
        if (row0 >= seq_q) {
            u.nblk[i] = 0;
        } else {
            const int last_row = min(row0 + kTileQ, seq_q) - 1;
            const int visible = causal ? min(seq_k, last_row + 1) : seq_k;
            u.nblk[i] = (visible + kTileKV - 1) / kTileKV;
        }
    }
    u.nmax = max(u.nblk[0], u.nblk[1]);
    return u;
}

template <int D, int STAGES, int EMU>
__global__ void __launch_bounds__(kWsThreads, 1)
fa_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ OMapSet tmap_o, int n_dst,
                 int seq_q, int seq_k, int heads, int q_pairs, int num_units, float scale_log2, int causal,
                 uint32_t* status) {
    using T = FaWsTraits<D, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;                                  // [2] query tiles
    const uint32_t ring_smem = q_smem + kQTiles * T::kTileBytes;        // [STAGES] K / V blocks
    const uint32_t o_smem = ring_smem + STAGES * T::kTileBytes;         // one O tile (staging for the TMA store)
    const uint32_t alpha_smem = o_smem + T::kTileBytes;                 // [2][128] fp32: factor for O_i, per row
    const uint32_t total_smem = alpha_smem + 2 * kTileQ * 4;            // [2][128] fp32: row sums of a finished unit
    const uint32_t bar_base = total_smem + 2 * kTileQ * 4;
    const uint32_t q_full = bar_base;                     // TMA -> MMA: the unit's Q tiles landed
    const uint32_t q_empty = q_full + 8;                  // MMA -> TMA: last S of the unit issued and complete
    const uint32_t kv_full = q_empty + 8;                 // [STAGES] TMA -> MMA
    const uint32_t kv_empty = kv_full + 8 * STAGES;       // [STAGES] MMA -> TMA
    const uint32_t s_full = kv_empty + 8 * STAGES;        // [2] MMA -> softmax: S_i ready
    const uint32_t p_full = s_full + 16;                  // [2][2] softmax -> MMA: half h of P_i written
    const uint32_t corr_full = p_full + 32;               // [2] softmax -> correction: factors of this block published
    const uint32_t o_ready = corr_full + 16;              // [2] correction -> MMA: O_i may be accumulated into
    const uint32_t o_final = o_ready + 16;                // [2] MMA -> correction: O_i of the unit complete
    const uint32_t sum_full = o_final + 16;               // [2] softmax -> correction: row sums published
    const uint32_t sum_empty = sum_full + 16;             // [2] correction -> softmax: row sums taken
    const uint32_t tmem_slot = sum_empty + 16;
    const uint32_t abort_slot = tmem_slot + 4;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
    volatile uint32_t* abort_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));
    float* alpha_ptr = reinterpret_cast<float*>(smem_aligned + (alpha_smem - smem_base));
    float* total_ptr = reinterpret_cast<float*>(smem_aligned + (total_smem - smem_base));
    const WaitGuard guard{abort_ptr, status};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    {
        // The layout above must fit behind the aligned base; it always does when the dynamic
        // segment starts on a 1024-byte boundary.  Otherwise report and leave (uniformly).
        uint32_t dyn_size;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
        if ((smem_base - smem_u32(smem_raw)) + static_cast<uint32_t>(T::kNeeded) > dyn_size) {
            if (threadIdx.x == 0) atomicCAS(status, 0u, 0x80000000u | 0x1fffu);
            return;
        }
    }

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(kv_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + 8 * i, 1);
            mbar_init(p_full + 16 * i, 8);       // one arrival per softmax warp of the tile
            mbar_init(p_full + 16 * i + 8, 8);
            mbar_init(corr_full + 8 * i, 8);
            mbar_init(o_ready + 8 * i, 4);       // one arrival per correction warp
            mbar_init(o_final + 8 * i, 1);
            mbar_init(sum_full + 8 * i, 8);
            mbar_init(sum_empty + 8 * i, 4);
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
        setmaxnreg_dec<kWsRegsLoadMma>();
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
            uint32_t o_ph[2] = {0, 0};
            bool ok = true;

            auto issue_s = [&](int i, uint32_t k_addr) {
                const uint32_t q_addr = q_smem + i * T::kTileBytes;
                if (!elect_one()) return;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
                    mma_ss<1>(tmem_base + T::kColS + i * kTileKV, smem_desc_kmajor_sw128(q_addr + off),
                              smem_desc_kmajor_sw128(k_addr + off), idesc_qk, kk > 0 ? 1u : 0u);
                }
            };
            // Half h of P V: 16-key steps [4h, 4h+4) of the block.  P: 16 keys = 8 packed columns.
            // V: 16 key rows = 2048 bytes; the second 64-wide span of the head dimension lives
            // one box (16 KiB) further.
            auto issue_pv_half = [&](int i, int h, uint32_t v_addr, bool accumulate) {
                if (!elect_one()) return;
#pragma unroll
                for (int kk = 4 * h; kk < 4 * h + 4; ++kk) {
                    mma_ts(tmem_base + T::kColO + i * D, tmem_base + T::kColS + i * kTileKV + kk * 8,
                           smem_desc_mnmajor_sw128(v_addr + kk * 2048, kBoxBytes), idesc_pv,
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

            for (int id = first_unit; id < num_units && ok; id += unit_stride) {
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
                        ok = wait(o_ready + 8 * i, o_ph[i], 0x1228u + i);
                        if (!ok) break;
                        o_ph[i] ^= 1u;
                        ok = wait(p_full + 16 * i, p_ph[i], 0x1230u + i);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv_half(i, 0, v_addr, j > 0);
                        ok = wait(p_full + 16 * i + 8, p_ph[i], 0x1238u + i);
                        if (!ok) break;
                        p_ph[i] ^= 1u;
                        tc_fence_after();
                        issue_pv_half(i, 1, v_addr, true);
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
        }
    } else if (warp < 8) {
        setmaxnreg_dec<kWsRegsCorrection>();
        // --------------------------------------------------------------- correction warpgroup
        const int quad = warp & 3;                      // tensor-memory lane quadrant
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        uint32_t c_ph[2] = {0, 0};                      // corr_full
        uint32_t u_ph[2] = {0, 0};                      // sum_full / o_final: one completion per unit the tile takes part in
        bool ok = true;
        // O_0 and O_1 start out free.
        if (lane == 0 && first_unit < num_units) {
            mbar_arrive(o_ready);
            mbar_arrive(o_ready + 8);
        }
        for (int id = first_unit; id < num_units && ok; id += unit_stride) {
            const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
            for (int j = 1; j < u.nmax && ok; ++j) {
                for (int i = 0; i < 2 && ok; ++i) {
                    if (j >= u.nblk[i]) continue;
                    ok = __all_sync(0xffffffffu, mbar_wait(guard, corr_full + 8 * i, c_ph[i], 0x1500u + i));
                    if (!ok) break;
                    c_ph[i] ^= 1u;
                    const float alpha = alpha_ptr[i * kTileQ + row_in_tile];
                    if (__any_sync(0xffffffffu, alpha != 1.f)) {
                        tc_fence_after();
                        const uint32_t t_o = tmem_base + lane_base + T::kColO + i * D;
#pragma unroll 1
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t o[32];
                            tmem_ld_32x32b_x32(t_o + c * 32, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
                            tmem_st_32x32b_x32(t_o + c * 32, o);
                        }
                        tmem_wait_st();
                        tc_fence_before();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_ready + 8 * i);
                }
            }
            // ---------------------------------------------------------------------- epilogue
            for (int i = 0; i < 2 && ok; ++i) {
                if (u.nblk[i] == 0) continue;
                ok = __all_sync(0xffffffffu, mbar_wait(guard, sum_full + 8 * i, u_ph[i], 0x1510u + i));
                if (!ok) break;
                const float l = total_ptr[i * kTileQ + row_in_tile];
                __syncwarp();
                if (lane == 0) mbar_arrive(sum_empty + 8 * i);
                ok = __all_sync(0xffffffffu, mbar_wait(guard, o_final + 8 * i, u_ph[i], 0x1518u + i));
                if (!ok) break;
                tc_fence_after();
                const float inv = (l == 0.f) ? 1.f : (1.f / l);
                const uint32_t t_o = tmem_base + lane_base + T::kColO + i * D;
                // the stores of the previous tile have read the staging rows of this warp
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32b_x32(t_o + c * 32, o);
                    tmem_wait_ld();
                    if (c == D / 32 - 1) {
                        // O_i is in registers: the next unit may overwrite it
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(o_ready + 8 * i);
                    }
                    uint32_t h[16];
#pragma unroll
                    for (int x = 0; x < 16; ++x)
                        h[x] = pack_f16x2(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
                    const uint32_t row_addr = o_smem + (c >> 1) * kBoxBytes + row_in_tile * 128;
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int chunk = (c & 1) * 4 + jj;
                        st_shared_v4(row_addr + ((chunk ^ (row_in_tile & 7)) << 4), h[4 * jj], h[4 * jj + 1],
                                     h[4 * jj + 2], h[4 * jj + 3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    // this warp's 32 rows of every 64-column box, to every destination
                    for (int d = 0; d < n_dst; ++d)
                        for (int b = 0; b < T::kBoxes; ++b)
                            tma_store_4d(&tmap_o.m[d], o_smem + b * kBoxBytes + quad * 32 * 128, b * 64,
                                         u.q0 + i * kTileQ + quad * 32, u.head, u.batch);
                    tma_store_commit();
                }
                u_ph[i] ^= 1u;
            }
        }
        if (lane == 0) tma_store_wait_all<0>();
    } else {
        setmaxnreg_inc<kWsRegsSoftmax>();
        // ------------------------------------------------------------------ softmax warps
        const int i = (warp - 8) >> 3;                  // query tile of this warp
        const int quad = warp & 3;                      // tensor-memory lane quadrant
        const int half = ((warp - 8) >> 2) & 1;         // which 16 lanes of the quadrant
        const int qt = lane & 3;                        // position in the quad: columns 2qt, 2qt+1 of every 8
        const int row_a = quad * 32 + half * 16 + (lane >> 2);   // rows of this thread inside the tile
        const int row_b = row_a + 8;
        const uint32_t t_s = tmem_base + (static_cast<uint32_t>(quad * 32 + half * 16) << 16) + T::kColS + i * kTileKV;
        const Exp2PolyConsts poly = make_exp2_poly_consts();
        const f32x2 scale2 = pack2(scale_log2, scale_log2);
        uint32_t s_ph = 0;
        uint32_t units_done = 0;
        bool ok = true;
        for (int id = first_unit; id < num_units && ok; id += unit_stride) {
            const UnitCoord u = unit_coord(id, q_pairs, heads, seq_q, seq_k, causal);
            const int n = u.nblk[i];
            if (n == 0) continue;
            const int grow_a = u.q0 + i * kTileQ + row_a;   // query index of row a in the sequence
            float m_a = -INFINITY, m_b = -INFINITY;         // running max the accumulators are scaled to
            f32x2 l_a = pack2(0.f, 0.f), l_b = pack2(0.f, 0.f);   // partial row sums (this thread's columns)
            for (int j = 0; j < n && ok; ++j) {
                ok = __all_sync(0xffffffffu, mbar_wait(guard, s_full + 8 * i, s_ph, 0x1300u + i));
                if (!ok) break;
                s_ph ^= 1u;
                tc_fence_after();
                const int col0 = j * kTileKV;
                const bool need_mask =
                    (col0 + kTileKV > seq_k) || (causal && (col0 + kTileKV - 1 > u.q0 + i * kTileQ));
                const int lim_a = causal ? min(seq_k - 1, grow_a) : (seq_k - 1);   // last visible key
                const int lim_b = causal ? min(seq_k - 1, grow_a + 8) : (seq_k - 1);
                // ------------------------------------------------ pass 1: row max
                float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t v[32];
                    tmem_ld_16x256b_x8(t_s + c * 64, v);
                    tmem_wait_ld();
                    if (need_mask) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const int col = col0 + c * 64 + 8 * k + 2 * qt;
                            if (col > lim_a) v[4 * k] = 0xff800000u;
                            if (col + 1 > lim_a) v[4 * k + 1] = 0xff800000u;
                            if (col > lim_b) v[4 * k + 2] = 0xff800000u;
                            if (col + 1 > lim_b) v[4 * k + 3] = 0xff800000u;
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        mx_a = max3(mx_a, __uint_as_float(v[4 * k]), __uint_as_float(v[4 * k + 1]));
                        mx_b = max3(mx_b, __uint_as_float(v[4 * k + 2]), __uint_as_float(v[4 * k + 3]));
                    }
                }
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                // Rescale only when the max moved enough to matter (always on the first block).
                const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
                const bool need_a = (mn_a - m_a) * scale_log2 > kRescaleLog2 || m_a == -INFINITY;
                const bool need_b = (mn_b - m_b) * scale_log2 > kRescaleLog2 || m_b == -INFINITY;
                float alpha_a = 1.f, alpha_b = 1.f;
                if (__any_sync(0xffffffffu, need_a || need_b)) {
                    if (need_a) {
                        alpha_a = (m_a == -INFINITY) ? 0.f : fast_exp2((m_a - mn_a) * scale_log2);
                        m_a = mn_a;
                        l_a = mul2(l_a, pack2(alpha_a, alpha_a));
                    }
                    if (need_b) {
                        alpha_b = (m_b == -INFINITY) ? 0.f : fast_exp2((m_b - mn_b) * scale_log2);
                        m_b = mn_b;
                        l_b = mul2(l_b, pack2(alpha_b, alpha_b));
                    }
                }
                if (j > 0) {
                    // publish the factors of this block for the correction warpgroup
                    if (qt == 0) {
                        alpha_ptr[i * kTileQ + row_a] = alpha_a;
                        alpha_ptr[i * kTileQ + row_b] = alpha_b;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(corr_full + 8 * i);
                }
                // ------------------------------------------------ pass 2: P = exp2(s*scale - m*scale)
                const float nm_a = -((m_a == -INFINITY) ? 0.f : m_a) * scale_log2;
                const float nm_b = -((m_b == -INFINITY) ? 0.f : m_b) * scale_log2;
                const f32x2 nm2_a = pack2(nm_a, nm_a), nm2_b = pack2(nm_b, nm_b);
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t v[32];
                    tmem_ld_16x256b_x8(t_s + c * 64, v);
                    tmem_wait_ld();
                    if (need_mask) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const int col = col0 + c * 64 + 8 * k + 2 * qt;
                            if (col > lim_a) v[4 * k] = 0xff800000u;
                            if (col + 1 > lim_a) v[4 * k + 1] = 0xff800000u;
                            if (col > lim_b) v[4 * k + 2] = 0xff800000u;
                            if (col + 1 > lim_b) v[4 * k + 3] = 0xff800000u;
                        }
                    }
                    uint32_t pr[16];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const f32x2 xs = fma2(pack2(__uint_as_float(v[4 * k + 2 * r]), __uint_as_float(v[4 * k + 2 * r + 1])),
                                                  scale2, r ? nm2_b : nm2_a);
                            f32x2 pp;
                            // EMU of every 4 pairs take the polynomial path, the rest the SFU.
                            if (((2 * k + r) & 3) < EMU) {
                                pp = exp2_poly2(xs, poly);
                            } else {
                                float x0, x1;
                                unpack2(xs, x0, x1);
                                pp = pack2(fast_exp2(x0), fast_exp2(x1));
                            }
                            if (r) l_b = add2(l_b, pp); else l_a = add2(l_a, pp);
                            float p0, p1;
                            unpack2(pp, p0, p1);
                            pr[2 * k + r] = pack_f16x2(p0, p1);
                        }
                    }
                    // 64 keys = 32 packed columns; the scores they replace are already consumed.
                    tmem_st_16x128b_x8(t_s + c * 32, pr);
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(p_full + 16 * i + 8 * c);
                }
            }
            if (!ok) break;
            // ------------------------------------------------ row sums of the finished unit
            float ta, tb, hi;
            unpack2(l_a, ta, hi);
            ta += hi;
            unpack2(l_b, tb, hi);
            tb += hi;
            ta += __shfl_xor_sync(0xffffffffu, ta, 1);
            tb += __shfl_xor_sync(0xffffffffu, tb, 1);
            ta += __shfl_xor_sync(0xffffffffu, ta, 2);
            tb += __shfl_xor_sync(0xffffffffu, tb, 2);
            if (units_done > 0) {
                // the correction warps have taken the previous unit's sums
                ok = __all_sync(0xffffffffu, mbar_wait(guard, sum_empty + 8 * i, (units_done - 1) & 1u, 0x1310u + i));
                if (!ok) break;
            }
            if (qt == 0) {
                total_ptr[i * kTileQ + row_a] = ta;
                total_ptr[i * kTileQ + row_b] = tb;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sum_full + 8 * i);
            ++units_done;
        }
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
