// Pieces shared by the attention kernels: tile constants, the set of output tensor maps and
// the scalar / packed-pair arithmetic helpers of the softmax.
#pragma once

#include <cmath>

#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kTileQ = 128;
constexpr int kTileKV = 128;
constexpr int kQTiles = 2;
constexpr int kBoxBytes = 128 * 128;      // one TMA box: 128 rows x 64 fp16 (128 bytes)
constexpr int kMaxDst = 8;                // copies of O one launch can write (one per GPU of a box)
constexpr float kRescaleLog2 = 8.0f;      // rescale O only when the max grew by > 2^8

// Tensor maps of every destination of O: one entry is plain attention; several make the
// epilogue store each finished tile into all of them (peers' memory over NVLink included),
// which leaves a head shard in every rank's full tensor without a separate all-gather.
struct OMapSet {
    CUtensorMap m[kMaxDst];
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Packed pairs of fp32 (one 64-bit register, two lanes of the FMA pipe per instruction).
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// 2^x for a pair, on the FMA and integer pipes instead of the SFU: x = n + f with n the
// nearest integer (magic-number rounding) and f in [-0.5, 0.5]; 2^f by a cubic whose
// coefficients minimise the maximum relative error on that interval (7.5e-5, below half an
// fp16 ulp, and P is rounded to fp16 right after); 2^n by adding n to the exponent field.
// x is clamped at -126 so the exponent cannot wrap (masked scores, -inf, become 2^-126).
struct Exp2PolyConsts {
    f32x2 magic, neg_magic, neg_one, c3, c2, c1, c0;
};
__device__ __forceinline__ Exp2PolyConsts make_exp2_poly_consts() {
    Exp2PolyConsts k;
    k.magic = pack2(12582912.f, 12582912.f);  // 1.5 * 2^23
    k.neg_magic = pack2(-12582912.f, -12582912.f);
    k.neg_one = pack2(-1.f, -1.f);
    k.c3 = pack2(0.0551716685f, 0.0551716685f);
    k.c2 = pack2(0.2426111251f, 0.2426111251f);
    k.c1 = pack2(0.6932609677f, 0.6932609677f);
    k.c0 = pack2(0.9999280572f, 0.9999280572f);
    return k;
}
__device__ __forceinline__ f32x2 exp2_poly2(f32x2 x, const Exp2PolyConsts& k) {
    float x0, x1;
    unpack2(x, x0, x1);
    const f32x2 xc = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
    const f32x2 xr = add2(xc, k.magic);          // integer part in the low mantissa bits
    const f32x2 n = add2(xr, k.neg_magic);
    const f32x2 f = fma2(n, k.neg_one, xc);      // x - n
    f32x2 p = fma2(k.c3, f, k.c2);
    p = fma2(p, f, k.c1);
    p = fma2(p, f, k.c0);
    float p0, p1, r0, r1;
    unpack2(p, p0, p1);
    unpack2(xr, r0, r1);
    // exponent += n: one integer multiply-add per element (n sits in the low bits of xr;
    // the bits of the magic constant vanish in the shift by 23)
    p0 = __int_as_float(__float_as_int(r0) * 8388608 + __float_as_int(p0));
    p1 = __int_as_float(__float_as_int(r1) * 8388608 + __float_as_int(p1));
    return pack2(p0, p1);
}

// (pair of the head, head, batch) of unit `id`, and the key blocks its two tiles visit.
struct UnitCoord {
    int q0, head, batch;
    int nblk[2];
    int nmax;
};
// Unit a persistent CTA works on in its k-th iteration, given its schedule slot
// first + k * stride.  Normally the slot itself; with causal = 2 a CTA takes two consecutive
// units at a time (a heavy and a light one of the same head, see unit_coord), so every CTA
// carries the same weight whatever the sequence length.
__device__ __forceinline__ int schedule_unit(int slot, int first, int stride, int causal) {
    if (causal != 2) return slot;
    const int k = (slot - first) / stride;
    return 2 * (first + (k >> 1) * stride) + (k & 1);
}
__device__ __forceinline__ UnitCoord unit_coord(int id, int q_pairs, int heads, int seq_q, int seq_k, int causal) {
    UnitCoord u;
    const int hb = id / q_pairs;
    const int p = id - hb * q_pairs;
    // causal = 1: heaviest units of a head first.  causal = 2 (schedule_unit's pairing): heavy and
    // light units of a head alternate (last pair, first pair, last but one, second, ...), so
    // that two consecutive units always have the same total weight
    const int pair = causal == 2 ? ((p & 1) ? (p >> 1) : (q_pairs - 1 - (p >> 1))) : causal ? (q_pairs - 1 - p) : p;
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

#ifdef B200_FA_PROFILE
// Cycle counters of CTA 0 (profiling builds only): [0..7] MMA warp, [8..15] softmax warp 8,
// [16..23] softmax warp 16, [24..31] correction warp 4.
__device__ unsigned long long g_fa_profile[32];
#define FA_PROF_DECL unsigned long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; unsigned long long prof_t = clock64();
#define FA_PROF(n) { const unsigned long long prof_now = clock64(); prof_acc[n] += prof_now - prof_t; prof_t = prof_now; }
#define FA_PROF_DUMP(base) if (blockIdx.x == 0 && lane == 0) { for (int x = 0; x < 8; ++x) g_fa_profile[(base) + x] = prof_acc[x]; }
#else
#define FA_PROF_DECL
#define FA_PROF(n) {}
#define FA_PROF_DUMP(base) {}
#endif

}  // namespace
}  // namespace b200
