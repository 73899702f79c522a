// GEMM config registry with the reference's shape: struct GemmConfig, kGemmConfigs[],
// kGemmConfigCount (gemm/gemm_config_registry.hpp.in:11-37 of HugeOrca/sm120-dl).  A caller
// written against the reference (its test harness reads .name, .bm, .bn, .bk and calls
// .run, gemm/test.cpp:449-465, 597-604) compiles against this header unchanged.
//
// Member names are the reference's; three of them carry Blackwell meanings:
//   stage    depth of the TMA -> MMA shared-memory ring
//   cwg      CTA group of the tcgen05.mma (1 = single CTA, 2 = CTA pair)
//   warps_m  cluster extent along M (= cwg);  warps_n  cluster extent along N (1)
//   bs_w     raster strip width in N-tiles
// and two trailing members are new: acc_bufs, tmem_cols.
//
// run(M,N,K,A,B,C,stream) computes C[M,N] = A[M,K] * B[N,K]^T (row-major, bf16, fp32
// accumulation, C overwritten) asynchronously on `stream` by calling the C ABI entry
// b200_gemm_bf16_tn.  Like the reference's gemm_tn (gemm/gemm_cute.hpp:288-291, 339-355)
// it prints to stderr and exits with status 1 on an unsupported shape or a CUDA error.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

// 2-byte bfloat16, convertible from/to float on the host (the reference uses
// cutlass::bfloat16_t, gemm/gemm_cute.hpp:28; the storage format is identical).
using bf16 = __nv_bfloat16;

struct GemmConfig {
    using RunFn = void (*)(
        int M,
        int N,
        int K,
        const bf16* A,
        const bf16* B,
        bf16* C,
        cudaStream_t stream);

    const char* name;
    int bm;
    int bn;
    int bk;
    int stage;
    int cwg;
    int warps_m;
    int warps_n;
    int bs_w;
    int smem_bytes;
    RunFn run;
    int acc_bufs;
    int tmem_cols;
};

extern const GemmConfig kGemmConfigs[];
extern const std::size_t kGemmConfigCount;
