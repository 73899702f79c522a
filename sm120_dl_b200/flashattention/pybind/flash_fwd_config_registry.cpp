// Table behind flash_fwd_config_registry.hpp and the per-config run functions (the
// counterpart of pybind/flash_fwd_config_registry.cu.in:3-8 and of run_flash_fwd_<cfg> /
// run_fixed_shape in pybind/flash_fwd_config.cu.in:22-91 of HugeOrca/sm120-dl).  Each run
// function allocates the output like the reference (empty_like(q)), uses scale
// 1/sqrt(head_dim), q's device and that device's current stream, and calls the C ABI
// entry b200_fa_fwd_fp16.  The head count is a run-time argument here, so every head count
// is accepted, not only the reference's {1,4,8,16,32,64,80}.
#include "flash_fwd_config_registry.hpp"

#include <cmath>
#include <cstring>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "b200dl.h"

namespace {

template <int Index>
torch::Tensor run_config(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, bool causal) {
    const b200_fa_config* cfg = b200_fa_get_config(Index);
    TORCH_CHECK(cfg != nullptr, "flash_fwd config ", Index, " is not in libb200dl.so");
    const int64_t head_dim = q.size(3);
    TORCH_CHECK(head_dim == cfg->head_dim, cfg->name, " expects head_dim=", cfg->head_dim, ", got ", head_dim);
    auto out = torch::empty_like(q);
    const float scale = 1.0f / std::sqrt(static_cast<float>(cfg->head_dim));
    c10::cuda::CUDAGuard device_guard(q.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream(q.get_device()).stream();
    const int64_t qs[3] = {q.stride(0), q.stride(1), q.stride(2)};
    const int64_t ks[3] = {k.stride(0), k.stride(1), k.stride(2)};
    const int64_t vs[3] = {v.stride(0), v.stride(1), v.stride(2)};
    const int64_t os[3] = {out.stride(0), out.stride(1), out.stride(2)};
    const int rc = b200_fa_fwd_fp16(Index, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                    static_cast<int>(q.size(0)), static_cast<int>(q.size(1)),
                                    static_cast<int>(k.size(1)), static_cast<int>(q.size(2)),
                                    static_cast<int>(head_dim), qs, ks, vs, os, scale, causal ? 1 : 0, stream);
    TORCH_CHECK(rc == B200_OK, "flashatten_v3 kernel launch failed: ", b200_last_error());
    return out;
}

int library_smem_bytes(int index, const char* name) {
    const b200_fa_config* c = b200_fa_get_config(index);
    TORCH_CHECK(c != nullptr && std::strcmp(c->name, name) == 0,
                "flash_fwd config registry out of step with libb200dl.so at entry ", index);
    return c->smem_bytes;
}

}  // namespace

#define B200_FA_ENTRY(INDEX, NAME, HEAD_DIM, BLOCK_M, BLOCK_N, NWARPS, STAGES) \
    FlashFwdConfig{NAME, HEAD_DIM, BLOCK_M, BLOCK_N, 2, 1, NWARPS, STAGES, library_smem_bytes(INDEX, NAME), \
                   &run_config<INDEX>},

const FlashFwdConfig kFlashFwdConfigs[] = {
#include "generated/flash_registry_entries.inc"
};
#undef B200_FA_ENTRY

const std::size_t kFlashFwdConfigCount = sizeof(kFlashFwdConfigs) / sizeof(kFlashFwdConfigs[0]);
const char* kFlashFwdDefaultConfigName = kFlashFwdConfigs[0].name;
