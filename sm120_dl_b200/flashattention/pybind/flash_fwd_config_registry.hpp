// Attention config registry with the reference's shape: struct FlashFwdConfig,
// kFlashFwdConfigs[], kFlashFwdConfigCount, kFlashFwdDefaultConfigName
// (flashattention/v3_mMnNkN/pybind/flash_fwd_config_registry.hpp.in:7-30 of
// HugeOrca/sm120-dl).  Member names are the reference's; block_m / block_n are the
// sequence-length granularity a config accepts (what check_runtime_shape tests), warps_m /
// warps_n hold the Blackwell tile split instead of an mma.sync warp grid: query tiles per
// CTA and 1.
#pragma once

#include <cstddef>

#include <torch/extension.h>

struct FlashFwdConfig {
    using RunFn = torch::Tensor (*)(
        const torch::Tensor& q,
        const torch::Tensor& k,
        const torch::Tensor& v,
        bool causal);

    const char* name;
    int head_dim;
    int block_m;
    int block_n;
    int warps_m;
    int warps_n;
    int nwarps;
    int stage;
    int smem_bytes;
    RunFn run;
};

extern const FlashFwdConfig kFlashFwdConfigs[];
extern const std::size_t kFlashFwdConfigCount;
extern const char* kFlashFwdDefaultConfigName;
