// Attention forward, layout "r1": one softmax thread per query row, rescale of O inside the
// softmax warps, one CTA per 256 query rows of a (batch, head).
//
//   warp 0  (1 thread)  TMA: Q tiles once, then K_0, V_0, K_1, V_1, ... into a STAGES-deep ring
//   warp 1  (elected    tcgen05.mma: S_i = Q_i K_j^T (smem x smem -> tensor memory) and
//            lane)      O_i += P_i V_j (P read from tensor memory, V MN-major from smem),
//                       interleaved so tile 1's MMAs run while tile 0's softmax runs
//   warps 4-7, 8-11     one softmax warpgroup per query tile, one thread per row: reads S_i
//                       from tensor memory, running max / sum in registers, writes P_i
//                       (fp16) over S_i, rescales O_i in tensor memory only when the row
//                       max grew by more than 2^kRescaleLog2; finally O_i / sum -> fp16 ->
//                       swizzled smem -> TMA store
//
// Tensor-memory columns: S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [256+D,256+2D).
#pragma once

#include "fa_common.cuh"

namespace b200 {
namespace {

constexpr int kFaThreads = 384;
// P V of a block is issued in two parts, 16-key MMA steps [0, kSplitP) and [kSplitP, 8): the
// first starts while the softmax warps still work on the remaining keys.  Measured on one
// box, B4 H32 S4096 D128 / B16 H32 S2048 D64, TFLOP/s: first part of 32 keys 1210 / 667,
// 64 keys 1194 / 665, 96 keys 1192 / 650, no split (kSplitP = 0) 1197 / 634.
constexpr int kSplitP = 2;
static_assert(kSplitP == 0 || kSplitP == 2 || kSplitP == 4 || kSplitP == 6, "parts end on 32-key chunks; 0 = one hand-off");
// Register budget after the role split.  setmaxnreg.inc blocks until the CTA's own pool
// (registers per thread at launch x threads) can supply the increase, so the two budgets
// must fit in what the CTA was launched with or the kernel never gets past the split.
constexpr int kRegsAtLaunch = 168;        // what ptxas assigns under __launch_bounds__(384, 1)
constexpr int kRegsLoadMma = 56;          // warps 0-3
constexpr int kRegsSoftmax = 224;         // warps 4-11
static_assert(kRegsLoadMma * 128 + kRegsSoftmax * 256 <= kRegsAtLaunch * kFaThreads,
              "setmaxnreg budgets exceed the registers the CTA is launched with");

template <int D, int STAGES>
struct FaTraits {
    static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
    static constexpr int kBoxes = D / 64;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a Q tile, a K block or a V block
    static constexpr int kNumBarriers = 1 + 2 * STAGES + 2 + 4;
    static constexpr int kSmemBytes = (kQTiles + STAGES) * kTileBytes + kNumBarriers * 8 + 16 + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0;
    static constexpr int kColO = 256;
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB shared-memory limit of sm_100");
};

template <int D, int STAGES, int EMU>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ OMapSet tmap_o, int n_dst,
              int seq_q, int seq_k, float scale_log2, int causal, uint32_t* status) {
    using T = FaTraits<D, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;                               // [2] query tiles (later O staging)
    const uint32_t ring_smem = smem_base + kQTiles * T::kTileBytes;  // [STAGES] K / V blocks
    const uint32_t bar_base = ring_smem + STAGES * T::kTileBytes;
    const uint32_t q_full = bar_base;                     // TMA -> MMA: both Q tiles landed
    const uint32_t kv_full = q_full + 8;                  // [STAGES] TMA -> MMA
    const uint32_t kv_empty = kv_full + 8 * STAGES;       // [STAGES] MMA -> TMA
    const uint32_t s_full = kv_empty + 8 * STAGES;        // [2] MMA -> softmax: S_i (or final O_i) ready
    const uint32_t p_full = s_full + 16;                  // [2][2] softmax -> MMA: part h of P_i written (and O_i rescaled)
    const uint32_t tmem_slot = p_full + 32;
    const uint32_t abort_slot = tmem_slot + 4;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
    volatile uint32_t* abort_ptr = reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));
    const WaitGuard guard{abort_ptr, status};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Work unit: query rows [q0, q0 + 256) of (head, batch).  Heaviest causal units first.
    const int q_pairs = gridDim.x;
    const int pair = causal ? (q_pairs - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    const int q0 = pair * (kQTiles * kTileQ);
    // Key blocks each tile has to visit.
    int nblk[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row0 = q0 + i * kTileQ;
        if (row0 >= seq_q) {
            nblk[i] = 0;
        } else {
            const int last_row = min(row0 + kTileQ, seq_q) - 1;
            const int visible = causal ? min(seq_k, last_row + 1) : seq_k;
            nblk[i] = (visible + kTileKV - 1) / kTileKV;
        }
    }
    const int nmax = max(nblk[0], nblk[1]);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(kv_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + 8 * i, 1);
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

    if (warp < 4) {
        setmaxnreg_dec<kRegsLoadMma>();
        if (warp == 0 && lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            uint32_t q_bytes = 0;
            for (int i = 0; i < 2; ++i) if (nblk[i] > 0) q_bytes += T::kTileBytes;
            mbar_arrive_expect_tx(q_full, q_bytes);
            for (int i = 0; i < 2; ++i) {
                if (nblk[i] == 0) continue;
                for (int b = 0; b < T::kBoxes; ++b) {
                    tma_load_4d(q_smem + i * T::kTileBytes + b * kBoxBytes, &tmap_q, q_full, b * 64,
                                q0 + i * kTileQ, head, batch);
                }
            }
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int e = 0; e < 2 * nmax && ok; ++e) {  // ring entries: K_0, V_0, K_1, V_1, ...
                ok = mbar_wait(guard, kv_empty + 8 * s, ph ^ 1u, 0x1100u + s);
                if (!ok) break;
                mbar_arrive_expect_tx(kv_full + 8 * s, T::kTileBytes);
                const CUtensorMap* tm = (e & 1) ? &tmap_v : &tmap_k;
                const int row = (e >> 1) * kTileKV;
                for (int b = 0; b < T::kBoxes; ++b) {
                    tma_load_4d(ring_smem + s * T::kTileBytes + b * kBoxBytes, tm, kv_full + 8 * s, b * 64,
                                row, head, batch);
                }
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer
            // The whole warp walks this code so that addresses and descriptors stay warp-uniform
            // (a tcgen05.mma issued from single-lane divergent code costs ~86 cycles of issue,
            // from uniform code ~74 for smem x smem and ~60 for tmem x smem operands, measured);
            // one elected lane issues the instructions.
            constexpr uint32_t idesc_qk = make_idesc_f16(kTileQ, kTileKV, /*fp16*/ 0, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(kTileQ, D, /*fp16*/ 0, 0, /*V is MN-major*/ 1);
            int s = 0;           // ring slot of the next entry to consume
            uint32_t ph = 0;
            uint32_t p_ph[2] = {0, 0};
            bool ok = true;

            // Descriptors are built once per operand tile; a step of 16 along the head dimension
            // (S) or of 16 key rows (P V) is a constant added to the address field, so one MMA
            // costs two 64-bit adds beside the instruction itself (the issuing warp shares its
            // scheduler with two softmax warps).
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
            // Part h of P V: 16-key steps [0,kSplitP) or [kSplitP,8) of the block.  P: 16 keys = 8 packed columns.
            // V: 16 key rows = 2048 bytes; the second 64-wide span of the head dimension lives
            // one box (16 KiB) further.
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

            ok = wait(q_full, 0, 0x1200u);
            // K_0
            uint32_t k_addr = 0, v_addr = 0;
            int k_slot = 0, v_slot = 0;
            if (ok && nmax > 0) {
                ok = wait(kv_full + 8 * s, ph, 0x1210u + s);
                k_addr = ring_smem + s * T::kTileBytes;
                k_slot = s;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                if (ok) {
                    tc_fence_after();
                    for (int i = 0; i < 2; ++i) {
                        if (nblk[i] > 0) {
                            issue_s(i, k_addr);
                            commit(s_full + 8 * i);
                        }
                    }
                    commit(kv_empty + 8 * k_slot);
                }
            }
            for (int j = 0; j < nmax && ok; ++j) {
                // V_j
                ok = wait(kv_full + 8 * s, ph, 0x1220u + s);
                if (!ok) break;
                v_addr = ring_smem + s * T::kTileBytes;
                v_slot = s;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                const bool more = (j + 1 < nmax);
                bool have_k = false;
                for (int i = 0; i < 2 && ok; ++i) {
                    if (j >= nblk[i]) continue;
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
                    if (j + 1 < nblk[i]) {
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
                    }
                    commit(s_full + 8 * i);
                }
                if (!ok) break;
                commit(kv_empty + 8 * v_slot);
                if (more) {
                    if (!have_k) {
                        // No tile needed K_{j+1} (cannot happen: nmax = max(nblk)); keep the ring in step.
                        ok = wait(kv_full + 8 * s, ph, 0x1250u + s);
                        k_slot = s;
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    commit(kv_empty + 8 * k_slot);
                }
            }
        }
    } else {
        setmaxnreg_inc<kRegsSoftmax>();
        // ------------------------------------------------------------- softmax warpgroups
        const int i = (warp - 4) >> 2;                 // query tile of this warpgroup
        const int quad = warp & 3;                     // tensor-memory lane quadrant
        const int row_in_tile = quad * 32 + lane;
        const int row = q0 + i * kTileQ + row_in_tile;  // query index in the sequence
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_s = tmem_base + lane_base + T::kColS + i * kTileKV;
        const uint32_t t_o = tmem_base + lane_base + T::kColO + i * D;
        const int n = nblk[i];
        const Exp2PolyConsts poly = make_exp2_poly_consts();
        float m = -INFINITY;  // running max the accumulators are scaled to
        float l0 = 0.f, l1 = 0.f;  // running sum of exp2(s*scale - m*scale), two partial sums
        bool ok = true;
        for (int j = 0; j < n && ok; ++j) {
            ok = mbar_wait(guard, s_full + 8 * i, j & 1, 0x1300u + i);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[4][32];
            tmem_ld_32x32b_x32(t_s + 0, sr[0]);
            tmem_ld_32x32b_x32(t_s + 32, sr[1]);
            tmem_ld_32x32b_x32(t_s + 64, sr[2]);
            tmem_ld_32x32b_x32(t_s + 96, sr[3]);
            tmem_wait_ld();
            const int col0 = j * kTileKV;
            const bool need_mask = (col0 + kTileKV > seq_k) || (causal && (col0 + kTileKV - 1 > q0 + i * kTileQ));
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
        const float l = l0 + l1;
        if (ok && n > 0) {
            // ------------------------------------------------------------------ epilogue
            ok = mbar_wait(guard, s_full + 8 * i, n & 1, 0x1310u + i);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after();
                const float inv = (l == 0.f) ? 1.f : (1.f / l);
                const uint32_t stage = q_smem + i * T::kTileBytes;  // Q_i is dead: reuse as O staging
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32b_x32(t_o + c * 32, o);
                    tmem_wait_ld();
                    uint32_t h[16];
#pragma unroll
                    for (int x = 0; x < 16; ++x)
                        h[x] = pack_f16x2(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
                    const uint32_t row_addr = stage + (c >> 1) * kBoxBytes + row_in_tile * 128;
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int chunk = (c & 1) * 4 + jj;
                        st_shared_v4(row_addr + ((chunk ^ (row_in_tile & 7)) << 4), h[4 * jj], h[4 * jj + 1],
                                     h[4 * jj + 2], h[4 * jj + 3]);
                    }
                }
                fence_proxy_async_smem();
                named_bar_sync(1 + i, kTileQ);
                if (row_in_tile == 0) {
                    for (int d = 0; d < n_dst; ++d)
                        for (int b = 0; b < T::kBoxes; ++b)
                            tma_store_4d(&tmap_o.m[d], stage + b * kBoxBytes, b * 64, q0 + i * kTileQ, head, batch);
                    tma_store_commit();
                    tma_store_wait_read<0>();   // shared memory may go; the writes finish on their own before the grid does
                }
            }
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
