// Thin C entry points around the reference project's own kernels, compiled from the
// reference's sources where they lie (they are found through -I at build time; none of
// them is copied here) for sm_100a.  TEST INFRASTRUCTURE ONLY: the result, a shared library
// under oracle/_ref/, is a same-box witness for the parity tests and a same-box baseline for
// the tables; nothing in the product or in the timed region of the benchmark loads it.
//
//   REF_UNIT_GEMM                 gemm_tn<bf16, ...> (gemm/gemm_cute.hpp:268-356), the two configs
//                                 the reference's README lists as best for large shapes
//   REF_UNIT_FA, REF_FA_D, REF_FA_H
//                                 flash_fwd<half_t, causal, H, D, ...>
//                                 (flashattention/v3_mMnNkN/flashatten_v3.hpp:536-573), the
//                                 README's best config of that head dimension
#include <cuda_runtime.h>

#if defined(REF_UNIT_GEMM)
#include "gemm_cute.hpp"

extern "C" int ref_gemm_bf16_tn(int which, int M, int N, int K, const void* A, const void* B, void* C, void* stream) {
    const bf16* a = static_cast<const bf16*>(A);
    const bf16* b = static_cast<const bf16*>(B);
    bf16* c = static_cast<bf16*>(C);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (which == 0) {
        // bf16_bm128_bn64_bk64_s3_cwg2_wm2_wn4_bsw8 (gemm/README.md:187)
        if (M % 128 || N % 64 || K % 64) return -2;
        gemm_tn<bf16, 128, 64, 64, 3, 2, 2, 4, 8>(M, N, K, a, b, c, s);
    } else if (which == 1) {
        // bf16_bm128_bn128_bk64_s2_cwg2_wm2_wn4_bsw8 (gemm/README.md:184-185)
        if (M % 128 || N % 128 || K % 64) return -2;
        gemm_tn<bf16, 128, 128, 64, 2, 2, 2, 4, 8>(M, N, K, a, b, c, s);
    } else {
        return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
#endif

#if defined(REF_UNIT_FA)
#include <cutlass/numeric_types.h>
#include "flashatten_v3.hpp"

#define REF_CAT2(a, b) a##b
#define REF_CAT(a, b) REF_CAT2(a, b)
#define REF_FA_NAME REF_CAT(REF_CAT(REF_CAT(ref_fa_fwd_fp16_d, REF_FA_D), _h), REF_FA_H)

// hd128_bm128_bn64_wm8_wn1_s2 / hd64_bm128_bn32_wm8_wn1_s2 (flashattention/v3_mMnNkN/README.md:402-419)
extern "C" int REF_FA_NAME(int causal, int batch, int seq, const void* q, const void* k, const void* v, void* o,
                           float scale, void* stream) {
    constexpr int kBlockN = REF_FA_D == 128 ? 64 : 32;
    if (seq % 128 != 0) return -2;
    using T = cutlass::half_t;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (causal) {
        flash_fwd<T, true, REF_FA_H, REF_FA_D, 128, kBlockN, 8, 1, 2>(scale, seq, batch, static_cast<const T*>(q),
                                                                       static_cast<const T*>(k), static_cast<const T*>(v),
                                                                       static_cast<T*>(o), s);
    } else {
        flash_fwd<T, false, REF_FA_H, REF_FA_D, 128, kBlockN, 8, 1, 2>(scale, seq, batch, static_cast<const T*>(q),
                                                                        static_cast<const T*>(k), static_cast<const T*>(v),
                                                                        static_cast<T*>(o), s);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
#endif
