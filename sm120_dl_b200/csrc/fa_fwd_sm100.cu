// FP16 FlashAttention forward for sm_100a: host launchers, config table and C ABI.
//
// Same contract as the reference's flash_fwd / flash_atten_v3_fwd
// (flashattention/v3_mMnNkN/flashatten_v3.hpp:390-573): O = softmax(Q K^T * scale) V per
// (batch, head) on [B,S,H,D] fp16 tensors.  Two kernel layouts implement it (the reference
// ships two warp layouts as well, v3_mMnNkN and v3_mMn1k1):
//
//   r2  fa_fwd_ws.cuh         persistent CTAs; load, MMA, softmax and correction warpgroups;
//                             two softmax threads per query row
//   r1  fa_fwd_rowthread.cuh  one CTA per 256 query rows; one softmax thread per row, which
//                             also rescales O
//
// Sequence lengths need not be multiples of the tile: TMA zero-fills rows past the end,
// the last key block is masked, and stores are clipped by the tensor map.
#include <cmath>
#include <cstring>

#include "fa_fwd_rowthread.cuh"
#include "fa_fwd_rowthread_persistent.cuh"
#include "fa_fwd_ws.cuh"
#include "runtime.h"

namespace b200 {
namespace {

// ------------------------------------------------------------------------- host launchers
using FaLaunchFn = int (*)(const DeviceInfo*, const b200_fa_config&, const void*, const void*, const void*,
                           void* const*, int, int, int, int, int, const int64_t*, const int64_t*, const int64_t*,
                           const int64_t*, float, int, cudaStream_t);

// Tensor map over a [batch, seq, head, dim] tensor: dimensions innermost-first
// (dim, seq, head, batch), box = 64 x box_rows x 1 x 1, 128-byte swizzle.
int make_tmap(CUtensorMap* out, const void* base, int batch, int seq, int heads, int dim,
              const int64_t* strides /* batch, seq, head */, int box_rows) {
    const uint64_t dims[4] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(seq),
                              static_cast<uint64_t>(heads), static_cast<uint64_t>(batch)};
    const uint64_t sb[3] = {static_cast<uint64_t>(strides[1]) * 2, static_cast<uint64_t>(strides[2]) * 2,
                            static_cast<uint64_t>(strides[0]) * 2};
    const uint32_t box[4] = {64, static_cast<uint32_t>(box_rows), 1, 1};
    return encode_tmap_2byte(out, base, 4, dims, sb, box, true);
}

int gcd_int(int a, int b) {
    while (b != 0) {
        const int t = a % b;
        a = b;
        b = t;
    }
    return a;
}

template <int D, int STAGES, int EMU>
int launch_fa_r1(const DeviceInfo* dev, const b200_fa_config& cfg, const void* q, const void* k, const void* v,
                 void* const* o_list, int n_dst, int batch, int seq_q, int seq_k, int heads, const int64_t* qs,
                 const int64_t* ks, const int64_t* vs, const int64_t* os, float softmax_scale, int causal,
                 cudaStream_t stream) {
    using T = FaTraits<D, STAGES>;
    auto kernel = fa_fwd_kernel<D, STAGES, EMU>;
    CUtensorMap tq, tk, tv;
    OMapSet to;
    std::memset(&to, 0, sizeof(to));
    if (int rc = make_tmap(&tq, q, batch, seq_q, heads, D, qs, 128)) return rc;
    if (int rc = make_tmap(&tk, k, batch, seq_k, heads, D, ks, 128)) return rc;
    if (int rc = make_tmap(&tv, v, batch, seq_k, heads, D, vs, 128)) return rc;
    for (int d = 0; d < n_dst; ++d) {
        if (int rc = make_tmap(&to.m[d], o_list[d], batch, seq_q, heads, D, os, 128)) return rc;
    }
    static bool attr_done[kMaxDevices] = {};
    if (int rc = set_smem_once(kernel, T::kSmemBytes, dev->device, attr_done, cfg.name)) return rc;
    const int q_pairs = (seq_q + kQTiles * kTileQ - 1) / (kQTiles * kTileQ);
    if (heads > 65535 || batch > 65535) return fail(B200_ESHAPE, "heads and batch must be <= 65535");
    const dim3 grid(static_cast<unsigned>(q_pairs), static_cast<unsigned>(heads), static_cast<unsigned>(batch));
    const float scale_log2 = softmax_scale * 1.4426950408889634f;
    kernel<<<grid, kFaThreads, T::kSmemBytes, stream>>>(tq, tk, tv, to, n_dst, seq_q, seq_k, scale_log2,
                                                        causal ? 1 : 0, dev->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200_ECUDA, "launch of %s failed: %s", cfg.name, cudaGetErrorString(e));
    return B200_OK;
}

template <int D, int STAGES, int EMU, int TPR>
int launch_fa_r2(const DeviceInfo* dev, const b200_fa_config& cfg, const void* q, const void* k, const void* v,
                 void* const* o_list, int n_dst, int batch, int seq_q, int seq_k, int heads, const int64_t* qs,
                 const int64_t* ks, const int64_t* vs, const int64_t* os, float softmax_scale, int causal,
                 cudaStream_t stream) {
    using T = FaWsTraits<D, STAGES>;
    auto kernel = fa_fwd_ws_kernel<D, STAGES, EMU, TPR>;
    CUtensorMap tq, tk, tv;
    OMapSet to;
    std::memset(&to, 0, sizeof(to));
    if (int rc = make_tmap(&tq, q, batch, seq_q, heads, D, qs, 128)) return rc;
    if (int rc = make_tmap(&tk, k, batch, seq_k, heads, D, ks, 128)) return rc;
    if (int rc = make_tmap(&tv, v, batch, seq_k, heads, D, vs, 128)) return rc;
    for (int d = 0; d < n_dst; ++d) {
        // each correction warp stores its own 32 rows of a finished tile
        if (int rc = make_tmap(&to.m[d], o_list[d], batch, seq_q, heads, D, os, 32)) return rc;
    }
    static bool attr_done[kMaxDevices] = {};
    if (int rc = set_smem_once(kernel, T::kSmemBytes, dev->device, attr_done, cfg.name)) return rc;
    const int q_pairs = (seq_q + kQTiles * kTileQ - 1) / (kQTiles * kTileQ);
    const long units = static_cast<long>(q_pairs) * heads * batch;
    if (units > 0x7fffffffL) return fail(B200_ESHAPE, "too many work units");
    int grid = dev->sm_count < units ? dev->sm_count : static_cast<int>(units);
    if (causal && units > grid) {
        // Units of a head are ordered heaviest first and CTAs take every grid-th unit: with a
        // grid coprime to the units per head every CTA meets every weight class equally often.
        while (grid > 1 && gcd_int(grid, q_pairs) != 1) --grid;
    }
    const float scale_log2 = softmax_scale * 1.4426950408889634f;
    kernel<<<grid, ws_threads(TPR), T::kSmemBytes, stream>>>(tq, tk, tv, to, n_dst, seq_q, seq_k, heads, q_pairs,
                                                        static_cast<int>(units), scale_log2, causal ? 1 : 0,
                                                        dev->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200_ECUDA, "launch of %s failed: %s", cfg.name, cudaGetErrorString(e));
    return B200_OK;
}

// Layout r4: the row-thread kernel with persistent CTAs.
template <int D, int STAGES, int EMU>
int launch_fa_r4(const DeviceInfo* dev, const b200_fa_config& cfg, const void* q, const void* k, const void* v,
                 void* const* o_list, int n_dst, int batch, int seq_q, int seq_k, int heads, const int64_t* qs,
                 const int64_t* ks, const int64_t* vs, const int64_t* os, float softmax_scale, int causal,
                 cudaStream_t stream) {
    using T = FaPersTraits<D, STAGES>;
    auto kernel = fa_fwd_pers_kernel<D, STAGES, EMU>;
    CUtensorMap tq, tk, tv;
    OMapSet to;
    std::memset(&to, 0, sizeof(to));
    if (int rc = make_tmap(&tq, q, batch, seq_q, heads, D, qs, 128)) return rc;
    if (int rc = make_tmap(&tk, k, batch, seq_k, heads, D, ks, 128)) return rc;
    if (int rc = make_tmap(&tv, v, batch, seq_k, heads, D, vs, 128)) return rc;
    for (int d = 0; d < n_dst; ++d) {
        if (int rc = make_tmap(&to.m[d], o_list[d], batch, seq_q, heads, D, os, 128)) return rc;
    }
    static bool attr_done[kMaxDevices] = {};
    if (int rc = set_smem_once(kernel, T::kSmemBytes, dev->device, attr_done, cfg.name)) return rc;
    const int q_pairs = (seq_q + kQTiles * kTileQ - 1) / (kQTiles * kTileQ);
    const long units = static_cast<long>(q_pairs) * heads * batch;
    if (units > 0x7fffffffL) return fail(B200_ESHAPE, "too many work units");
    int grid = dev->sm_count < units ? dev->sm_count : static_cast<int>(units);
    // Causal units differ in weight.  With many units per CTA and long sequences a CTA takes them
    // in pairs of one heavy and one light unit of a head, equal in total (mode 2); otherwise
    // heaviest first with a grid coprime to the units per head, so that every CTA meets every
    // weight class (mode 1).  Measured, mode 1 / mode 2 (ms): B2 H64 S4096 D128 0.516 / 0.486,
    // B1 H32 S16384 2.33 / 1.77, but B1 H32 S8192 (7 units per CTA: pairs halve the granularity)
    // 0.531 / 0.571 and B8 H32 S2048 D64 (8 units per head, the light ones one or two blocks
    // long: with pairs every CTA is in its short units at the same time) 0.250 / 0.287.
    int causal_mode = causal ? 1 : 0;
    if (causal && units >= 12L * grid && q_pairs % 2 == 0 && q_pairs >= 16) {
        causal_mode = 2;
    } else if (causal && units > grid) {
        while (grid > 1 && gcd_int(grid, q_pairs) != 1) --grid;
    }
    const float scale_log2 = softmax_scale * 1.4426950408889634f;
    kernel<<<grid, kFaThreads, T::kSmemBytes, stream>>>(tq, tk, tv, to, n_dst, seq_q, seq_k, heads, q_pairs,
                                                        static_cast<int>(units), scale_log2, causal_mode,
                                                        dev->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200_ECUDA, "launch of %s failed: %s", cfg.name, cudaGetErrorString(e));
    return B200_OK;
}

template <int D, int STAGES, int EMU, int LAYOUT>
constexpr FaLaunchFn fa_launcher() {
    static_assert(LAYOUT >= 1 && LAYOUT <= 4,
                  "layouts: 1 row-thread, 2 and 3 warp-specialised with 2 and 1 softmax threads per row, 4 persistent row-thread");
    if constexpr (LAYOUT == 2) return &launch_fa_r2<D, STAGES, EMU, 2>;
    else if constexpr (LAYOUT == 3) return &launch_fa_r2<D, STAGES, EMU, 1>;
    else if constexpr (LAYOUT == 4) return &launch_fa_r4<D, STAGES, EMU>;
    else return &launch_fa_r1<D, STAGES, EMU>;
}
template <int D, int STAGES, int LAYOUT>
constexpr int fa_smem_bytes() {
    if constexpr (LAYOUT == 4) return FaPersTraits<D, STAGES>::kSmemBytes;
    else if constexpr (LAYOUT >= 2) return FaWsTraits<D, STAGES>::kSmemBytes;
    else return FaTraits<D, STAGES>::kSmemBytes;
}

struct FaEntry {
    b200_fa_config cfg;
    FaLaunchFn launch;
};

#define B200_FA_CONFIG(NAME, D, STAGES, EMU, LAYOUT, BLOCK_M, BLOCK_N)                                        \
    FaEntry{b200_fa_config{NAME, D, BLOCK_M, BLOCK_N, kTileQ, kQTiles, kTileKV, STAGES,                        \
                           (LAYOUT == 2 ? ws_threads(2) : LAYOUT == 3 ? ws_threads(1) : kFaThreads) / 32, fa_smem_bytes<D, STAGES, LAYOUT>(),   \
                           LAYOUT},                                                                            \
            fa_launcher<D, STAGES, EMU, LAYOUT>()},

const FaEntry kFaEntries[] = {
#include "generated/flash_configs.inc"
};
#undef B200_FA_CONFIG

constexpr int kNumFaEntries = static_cast<int>(sizeof(kFaEntries) / sizeof(kFaEntries[0]));

}  // namespace
}  // namespace b200

extern "C" {

int b200_fa_num_configs(void) { return b200::kNumFaEntries; }

const b200_fa_config* b200_fa_get_config(int idx) {
    if (idx < 0 || idx >= b200::kNumFaEntries) return nullptr;
    return &b200::kFaEntries[idx].cfg;
}

int b200_fa_find_config(const char* name) {
    if (name == nullptr) return -1;
    for (int i = 0; i < b200::kNumFaEntries; ++i)
        if (std::strcmp(name, b200::kFaEntries[i].cfg.name) == 0) return i;
    return -1;
}

int b200_fa_default_config(int head_dim) {
    // The first generated config of a head dimension is its default (the generator orders them).
    for (int i = 0; i < b200::kNumFaEntries; ++i)
        if (b200::kFaEntries[i].cfg.head_dim == head_dim) return i;
    return -1;
}

int b200_fa_fwd_fp16_scatter(int config, const void* q, const void* k, const void* v, void* const* o_list, int n_dst,
                             int batch, int seq_q, int seq_k, int heads, int head_dim, const int64_t q_strides[3],
                             const int64_t k_strides[3], const int64_t v_strides[3], const int64_t o_strides[3],
                             float softmax_scale, int causal, void* stream) {
    using namespace b200;
    if (config < 0 || config >= kNumFaEntries) return fail(B200_EINVAL, "unknown attention config index %d", config);
    const FaEntry& e = kFaEntries[config];
    if (!q || !k || !v || !o_list) return fail(B200_EINVAL, "null tensor pointer");
    if (n_dst < 1 || n_dst > kMaxDst) return fail(B200_EINVAL, "n_dst must be 1..%d (got %d)", kMaxDst, n_dst);
    for (int d = 0; d < n_dst; ++d)
        if (!o_list[d]) return fail(B200_EINVAL, "null tensor pointer");
    if (!q_strides || !k_strides || !v_strides || !o_strides) return fail(B200_EINVAL, "null stride array");
    if (head_dim != e.cfg.head_dim)
        return fail(B200_ESHAPE, "%s expects head_dim=%d, got %d", e.cfg.name, e.cfg.head_dim, head_dim);
    if (batch <= 0 || heads <= 0 || seq_q <= 0 || seq_k <= 0)
        return fail(B200_ESHAPE, "batch, heads and sequence lengths must be positive");
    if (causal && seq_q != seq_k) return fail(B200_ESHAPE, "causal attention needs seq_q == seq_k");
    if (seq_q % e.cfg.block_m != 0) return fail(B200_ESHAPE, "seq_len must be a multiple of %d", e.cfg.block_m);
    if (seq_k % e.cfg.block_n != 0) return fail(B200_ESHAPE, "seq_len must be a multiple of %d", e.cfg.block_n);
    const int64_t* all[4] = {q_strides, k_strides, v_strides, o_strides};
    for (int t = 0; t < 4; ++t)
        for (int d = 0; d < 3; ++d)
            if (all[t][d] <= 0 || all[t][d] % 8 != 0)
                return fail(B200_EINVAL, "strides must be positive multiples of 8 elements");
    const DeviceInfo* dev = current_device();
    if (dev == nullptr) return B200_ENODEVICE;
    return e.launch(dev, e.cfg, q, k, v, o_list, n_dst, batch, seq_q, seq_k, heads, q_strides, k_strides, v_strides,
                    o_strides, softmax_scale, causal, static_cast<cudaStream_t>(stream));
}

int b200_fa_fwd_fp16(int config, const void* q, const void* k, const void* v, void* o, int batch, int seq_q,
                     int seq_k, int heads, int head_dim, const int64_t q_strides[3], const int64_t k_strides[3],
                     const int64_t v_strides[3], const int64_t o_strides[3], float softmax_scale, int causal,
                     void* stream) {
    if (!o) return b200::fail(B200_EINVAL, "null tensor pointer");
    return b200_fa_fwd_fp16_scatter(config, q, k, v, &o, 1, batch, seq_q, seq_k, heads, head_dim, q_strides, k_strides,
                                    v_strides, o_strides, softmax_scale, causal, stream);
}

#ifdef B200_FA_PROFILE
// Profiling builds only: the cycle counters CTA 0 of the last r2 launch recorded.
int b200_fa_profile_read(unsigned long long* out32) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out32, b200::g_fa_profile, 32 * sizeof(unsigned long long));
    return e == cudaSuccess ? B200_OK : b200::fail(B200_ECUDA, "reading the profile counters: %s", cudaGetErrorString(e));
}
#endif

}  // extern "C"
