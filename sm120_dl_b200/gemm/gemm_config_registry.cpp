// Table behind gemm_config_registry.hpp: one entry and one run wrapper per generated
// config (the counterpart of gemm/gemm_config_registry.cu.in:6-10 and the per-config
// instantiation units gemm/gemm.cu.in:59-66 of HugeOrca/sm120-dl).  Entries come from
// generated/gemm_registry_entries.inc, written by gemm_configs.py in the same order as
// the table inside libb200dl.so, so entry i runs library config i; the names are
// cross-checked once at start-up.
#include "gemm_config_registry.hpp"

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "b200dl.h"

namespace {

template <int Index>
void run_config(int M, int N, int K, const bf16* A, const bf16* B, bf16* C, cudaStream_t stream) {
    // The reference's gemm_tn refuses shapes its tile does not divide (gemm/gemm_cute.hpp:288-291).
    const b200_gemm_config* cfg = b200_gemm_get_config(Index);
    if (cfg == nullptr || M % cfg->bm != 0 || N % cfg->bn != 0 || K % cfg->bk != 0) {
        std::fprintf(stderr, "gemm_tn: M=%d N=%d K=%d must be multiples of BM=%d BN=%d BK=%d\n", M, N, K,
                     cfg ? cfg->bm : 0, cfg ? cfg->bn : 0, cfg ? cfg->bk : 0);
        std::exit(1);
    }
    const int rc = b200_gemm_bf16_tn(Index, M, N, K, A, K, B, K, C, N, stream);
    if (rc != B200_OK) {
        std::fprintf(stderr, "gemm_tn config %d failed (%d): %s\n", Index, rc, b200_last_error());
        std::exit(1);
    }
}

int library_smem_bytes(int index, const char* name) {
    const b200_gemm_config* c = b200_gemm_get_config(index);
    if (c == nullptr || std::strcmp(c->name, name) != 0) {
        std::fprintf(stderr, "config registry out of step with libb200dl.so at entry %d (%s vs %s)\n", index, name,
                     c ? c->name : "<none>");
        std::exit(1);
    }
    return c->smem_bytes;
}

int library_tmem_cols(int index) {
    const b200_gemm_config* c = b200_gemm_get_config(index);
    return c ? c->tmem_cols : 0;
}

}  // namespace

#define B200_GEMM_ENTRY(INDEX, NAME, BM, BN, BK, STAGES, CTA_GROUP, ACC_BUFS, BS_W)                    \
    GemmConfig{NAME, BM, BN, BK, STAGES, CTA_GROUP, CTA_GROUP, 1, BS_W, library_smem_bytes(INDEX, NAME), \
               &run_config<INDEX>, ACC_BUFS, library_tmem_cols(INDEX)},

const GemmConfig kGemmConfigs[] = {
#include "generated/gemm_registry_entries.inc"
};
#undef B200_GEMM_ENTRY

const std::size_t kGemmConfigCount = sizeof(kGemmConfigs) / sizeof(kGemmConfigs[0]);
