// Host-side plumbing shared by the GEMM and attention launchers: error reporting for the
// C ABI, per-device facts (SM count, compute capability, the kernel status word) and the
// TMA descriptor encoder fetched from the driver at run time (no link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200dl.h"

namespace b200 {

// Records a message for b200_last_error() and returns `code` so callers can `return fail(...)`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int max_smem_optin = 0;
    uint32_t* status = nullptr;  // one zero-initialised word block in device memory
    bool may_allocate = true;    // false for the allocation-free entry point: no stream-ordered workspace
};

// Facts about the CURRENT device (the reference hard-codes device 0 for its SM-count query,
// gemm/gemm_cute.hpp:343-346; a multi-GPU caller needs the current one).  nullptr + error
// message on failure.
const DeviceInfo* current_device();

constexpr int kMaxDevices = 64;

// SM count of the current device, or 0 when there is none; allocates nothing.
int current_sm_count();

// cudaFuncAttributeMaxDynamicSharedMemorySize, set once per (kernel, device); `done` is the
// caller's per-kernel table.  Safe to call from several host threads.
int set_smem_attribute_once(const void* kernel, int smem_bytes, int device, bool* done, const char* name);
template <typename Kernel>
int set_smem_once(Kernel kernel, int smem_bytes, int device, bool (&done)[kMaxDevices], const char* name) {
    return set_smem_attribute_once(reinterpret_cast<const void*>(kernel), smem_bytes, device, done, name);
}

// Encodes a tiled tensor map for 2-byte elements.  dims/strides are innermost-first;
// strides_bytes[i] is the byte stride of dimension i+1 (dimension 0 is contiguous).
// Returns 0 or a negative B200_E* code.
int encode_tmap_2byte(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

}  // namespace b200
