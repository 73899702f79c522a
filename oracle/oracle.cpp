// CPU oracle for the two hot paths.  TEST INFRASTRUCTURE ONLY: nothing in the product
// (the package, the C ABI library, the harnesses) may call into this file; only tests/,
// the smoke check and the cpu_baseline / reference legs of bench.py do.
//
// Parity status: the reference (HugeOrca/sm120-dl) holds NO golden vectors, fixtures or
// CPU implementation for either path -- its checks compare against cuBLAS
// (gemm/test.cpp:131-163, 394-420) and flash-attn (flashattention/v3_mMnNkN/verify.py:129)
// on the GPU at run time.  This oracle is therefore pinned against independent CPU
// implementations (numpy float64 / torch CPU; fixtures under tests/golden/) and is
// "parity unpinned" with respect to reference-held vectors, because none exist.
//
// What it restates:
//   GEMM       C[m,n] = sum_k A[m,k] * B[n,k]; A [M,K], B [N,K], C [M,N] row-major
//              (operand views at gemm/gemm_cute.hpp:302-304); bf16 operands widened
//              exactly, accumulation in double (the kernel accumulates in fp32 and rounds
//              the result to bf16, gemm/gemm_cute.hpp:233-238).
//   attention  O = softmax(Q K^T * scale) V per (batch, head) on [B,S,H,D] tensors
//              (4-D view at flashattention/v3_mMnNkN/kernel_traits.hpp:146-160, scale
//              1/sqrt(D) at pybind/flash_fwd_config.cu.in:27); causal rule "row < col is
//              masked" (flashatten_v3.hpp:101-103); fp16 operands widened exactly, scores,
//              max-subtracted softmax and the P V product in fp32, row sum in double,
//              fp32 output.
//   compare    the reference's pass rule |got-ref| <= abs + rel*|ref| with max_abs /
//              max_rel tracking (verify_result, gemm/test.cpp:165-230).
//
// Build: see oracle/Makefile (g++ -O3 -fopenmp, x86-64-v3 so the prebuilt library runs on
// any recent host).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float bf16_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

inline float fp16_to_f32(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {  // subnormal: renormalise
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            u = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// 4 x 4 block of dot products over K, both operands K-contiguous doubles.
inline void dot_block_4x4(const double* a, int64_t lda, const double* b, int64_t ldb, int K,
                          double out[4][4]) {
    double acc[4][4] = {};
    const double* a0 = a;
    const double* a1 = a + lda;
    const double* a2 = a + 2 * lda;
    const double* a3 = a + 3 * lda;
    const double* b0 = b;
    const double* b1 = b + ldb;
    const double* b2 = b + 2 * ldb;
    const double* b3 = b + 3 * ldb;
    double s00 = 0, s01 = 0, s02 = 0, s03 = 0, s10 = 0, s11 = 0, s12 = 0, s13 = 0;
    double s20 = 0, s21 = 0, s22 = 0, s23 = 0, s30 = 0, s31 = 0, s32 = 0, s33 = 0;
#pragma omp simd reduction(+ : s00, s01, s02, s03, s10, s11, s12, s13, s20, s21, s22, s23, s30, s31, s32, s33)
    for (int k = 0; k < K; ++k) {
        const double x0 = a0[k], x1 = a1[k], x2 = a2[k], x3 = a3[k];
        const double y0 = b0[k], y1 = b1[k], y2 = b2[k], y3 = b3[k];
        s00 += x0 * y0; s01 += x0 * y1; s02 += x0 * y2; s03 += x0 * y3;
        s10 += x1 * y0; s11 += x1 * y1; s12 += x1 * y2; s13 += x1 * y3;
        s20 += x2 * y0; s21 += x2 * y1; s22 += x2 * y2; s23 += x2 * y3;
        s30 += x3 * y0; s31 += x3 * y1; s32 += x3 * y2; s33 += x3 * y3;
    }
    acc[0][0] = s00; acc[0][1] = s01; acc[0][2] = s02; acc[0][3] = s03;
    acc[1][0] = s10; acc[1][1] = s11; acc[1][2] = s12; acc[1][3] = s13;
    acc[2][0] = s20; acc[2][1] = s21; acc[2][2] = s22; acc[2][3] = s23;
    acc[3][0] = s30; acc[3][1] = s31; acc[3][2] = s32; acc[3][3] = s33;
    std::memcpy(out, acc, sizeof(acc));
}

}  // namespace

extern "C" {

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline wants every core.
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// C (double, leading dimension ldc) = A * B^T for rows [row_begin, row_begin + row_count)
// of A.  A, B are raw bf16 bit patterns.  C is indexed C[(m - row_begin) * ldc + n].
void oracle_gemm_bf16_tn_f64(int M, int N, int K, const uint16_t* A, int64_t lda,
                             const uint16_t* B, int64_t ldb, double* C, int64_t ldc,
                             int row_begin, int row_count) {
    (void)M;
    constexpr int KC = 1024;  // K panel kept in cache: (RB + NB) * KC * 8 bytes
    constexpr int RB = 64;
    constexpr int NB = 64;
    for (int64_t i = 0; i < static_cast<int64_t>(row_count) * ldc; ++i) C[i] = 0.0;
    const int row_blocks = (row_count + RB - 1) / RB;
    const int col_blocks = (N + NB - 1) / NB;
#pragma omp parallel
    {
        std::vector<double> pa(static_cast<size_t>(RB) * KC), pb(static_cast<size_t>(NB) * KC);
#pragma omp for collapse(2) schedule(dynamic)
        for (int rb = 0; rb < row_blocks; ++rb) {
            for (int cb = 0; cb < col_blocks; ++cb) {
                const int r0 = rb * RB, r1 = std::min(row_count, r0 + RB);
                const int c0 = cb * NB, c1 = std::min(N, c0 + NB);
                for (int k0 = 0; k0 < K; k0 += KC) {
                    const int kc = std::min(KC, K - k0);
                    // zero-padded panels so the 4x4 micro-kernel never reads out of range
                    std::fill(pa.begin(), pa.end(), 0.0);
                    std::fill(pb.begin(), pb.end(), 0.0);
                    for (int r = r0; r < r1; ++r) {
                        const uint16_t* src = A + static_cast<int64_t>(row_begin + r) * lda + k0;
                        double* dst = pa.data() + static_cast<size_t>(r - r0) * KC;
                        for (int k = 0; k < kc; ++k) dst[k] = bf16_to_f32(src[k]);
                    }
                    for (int c = c0; c < c1; ++c) {
                        const uint16_t* src = B + static_cast<int64_t>(c) * ldb + k0;
                        double* dst = pb.data() + static_cast<size_t>(c - c0) * KC;
                        for (int k = 0; k < kc; ++k) dst[k] = bf16_to_f32(src[k]);
                    }
                    for (int r = r0; r < r1; r += 4) {
                        for (int c = c0; c < c1; c += 4) {
                            double blk[4][4];
                            dot_block_4x4(pa.data() + static_cast<size_t>(r - r0) * KC, KC,
                                          pb.data() + static_cast<size_t>(c - c0) * KC, KC, kc, blk);
                            for (int i = 0; i < 4 && r + i < r1; ++i)
                                for (int j = 0; j < 4 && c + j < c1; ++j)
                                    C[static_cast<int64_t>(r + i) * ldc + (c + j)] += blk[i][j];
                        }
                    }
                }
            }
        }
    }
}

// Attention forward for the query rows listed in `rows` (n_rows of them, each in
// [0, seq_q)) of every (batch, head).  q/k/v are raw fp16 bit patterns addressed with
// element strides {batch, seq, head} (dim stride 1).  out is fp32, laid out
// [batch][n_rows][head][dim] contiguous.  rows == nullptr means all rows 0..seq_q-1.
void oracle_fa_fwd_f32(int batch, int seq_q, int seq_k, int heads, int dim, const uint16_t* q,
                       const int64_t* qs, const uint16_t* k, const int64_t* ks,
                       const uint16_t* v, const int64_t* vs, float scale, int causal,
                       const int32_t* rows, int n_rows, float* out) {
    const int nr = rows ? n_rows : seq_q;
#pragma omp parallel
    {
        std::vector<float> kf(static_cast<size_t>(seq_k) * dim), vf(static_cast<size_t>(seq_k) * dim);
        std::vector<float> scores(seq_k), qf(dim), acc(dim);
#pragma omp for collapse(2) schedule(dynamic)
        for (int b = 0; b < batch; ++b) {
            for (int h = 0; h < heads; ++h) {
                for (int j = 0; j < seq_k; ++j) {
                    const uint16_t* kp = k + b * ks[0] + j * ks[1] + h * ks[2];
                    const uint16_t* vp = v + b * vs[0] + j * vs[1] + h * vs[2];
                    for (int d = 0; d < dim; ++d) {
                        kf[static_cast<size_t>(j) * dim + d] = fp16_to_f32(kp[d]);
                        vf[static_cast<size_t>(j) * dim + d] = fp16_to_f32(vp[d]);
                    }
                }
                for (int ri = 0; ri < nr; ++ri) {
                    const int i = rows ? rows[ri] : ri;
                    const uint16_t* qp = q + b * qs[0] + static_cast<int64_t>(i) * qs[1] + h * qs[2];
                    for (int d = 0; d < dim; ++d) qf[d] = fp16_to_f32(qp[d]);
                    const int limit = causal ? std::min(seq_k, i + 1) : seq_k;  // key j visible iff j <= i
                    float m = -std::numeric_limits<float>::infinity();
                    for (int j = 0; j < limit; ++j) {
                        const float* kr = kf.data() + static_cast<size_t>(j) * dim;
                        float s = 0.f;
#pragma omp simd reduction(+ : s)
                        for (int d = 0; d < dim; ++d) s += qf[d] * kr[d];
                        s *= scale;
                        scores[j] = s;
                        m = std::max(m, s);
                    }
                    double denom = 0.0;
                    std::fill(acc.begin(), acc.end(), 0.f);
                    for (int j = 0; j < limit; ++j) {
                        const float p = std::exp(scores[j] - m);
                        denom += p;
                        const float* vr = vf.data() + static_cast<size_t>(j) * dim;
#pragma omp simd
                        for (int d = 0; d < dim; ++d) acc[d] += p * vr[d];
                    }
                    const float inv = denom > 0.0 ? static_cast<float>(1.0 / denom) : 1.f;
                    float* op = out + ((static_cast<int64_t>(b) * nr + ri) * heads + h) * dim;
                    for (int d = 0; d < dim; ++d) op[d] = acc[d] * inv;
                }
            }
        }
    }
}

// Element-wise comparison with the reference's mixed tolerance.  got/ref are n doubles.
// stats: [0] max_abs, [1] max_rel (|diff| / max(|ref|, 1e-6) like the harnesses print),
// [2] index of the first mismatch or -1, [3] max |ref|, [4] rms(ref),
// [5] max |diff| / max(|ref_i|, rms(ref))  (the bounded relative error used for the
// "max relative error <= 1e-2" criterion).  Returns the mismatch count; non-finite values
// in got count as mismatches.
int64_t oracle_compare(const double* got, const double* ref, int64_t n, double abs_tol,
                       double rel_tol, double* stats) {
    double sumsq = 0.0, max_ref = 0.0;
#pragma omp parallel for reduction(+ : sumsq) reduction(max : max_ref)
    for (int64_t i = 0; i < n; ++i) {
        sumsq += ref[i] * ref[i];
        max_ref = std::max(max_ref, std::fabs(ref[i]));
    }
    const double rms = n > 0 ? std::sqrt(sumsq / static_cast<double>(n)) : 0.0;
    double max_abs = 0.0, max_rel = 0.0, max_brel = 0.0;
    int64_t bad = 0, first = std::numeric_limits<int64_t>::max();
#pragma omp parallel for reduction(max : max_abs, max_rel, max_brel) reduction(+ : bad) reduction(min : first)
    for (int64_t i = 0; i < n; ++i) {
        const double g = got[i], r = ref[i];
        const double d = std::isfinite(g) ? std::fabs(g - r) : std::numeric_limits<double>::infinity();
        max_abs = std::max(max_abs, d);
        max_rel = std::max(max_rel, d / std::max(std::fabs(r), 1e-6));
        max_brel = std::max(max_brel, d / std::max(std::fabs(r), std::max(rms, 1e-30)));
        if (!(d <= abs_tol + rel_tol * std::fabs(r))) {
            ++bad;
            first = std::min(first, i);
        }
    }
    stats[0] = max_abs;
    stats[1] = max_rel;
    stats[2] = bad ? static_cast<double>(first) : -1.0;
    stats[3] = max_ref;
    stats[4] = rms;
    stats[5] = max_brel;
    return bad;
}

}  // extern "C"
