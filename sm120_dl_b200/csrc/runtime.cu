// Host runtime of libb200dl.so: error strings, per-device state, TMA descriptor encoding.
#include "runtime.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace b200 {

namespace {

thread_local char t_error[512] = "";

DeviceInfo g_devices[kMaxDevices];
bool g_device_ready[kMaxDevices] = {};
std::mutex g_mutex;

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}

const DeviceInfo* current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        fail(B200_ENODEVICE, "cudaGetDevice failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        fail(B200_ENODEVICE, "device index %d out of range", dev);
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_device_ready[dev]) return &g_devices[dev];
    DeviceInfo info;
    info.device = dev;
    if ((e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) {
        fail(B200_ECUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    if (info.cc_major != 10) {
        fail(B200_ENODEVICE, "device %d has compute capability %d.x; this library contains sm_100a code only",
             dev, info.cc_major);
        return nullptr;
    }
    if ((e = cudaMalloc(reinterpret_cast<void**>(&info.status), 256)) != cudaSuccess ||
        (e = cudaMemset(info.status, 0, 256)) != cudaSuccess) {
        fail(B200_ECUDA, "allocating the status word failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    g_devices[dev] = info;
    g_device_ready[dev] = true;
    return &g_devices[dev];
}

int current_sm_count() {
    int dev = -1, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

int set_smem_attribute_once(const void* kernel, int smem_bytes, int device, bool* done, const char* name) {
    static std::mutex mu;
    if (device < 0 || device >= kMaxDevices) return fail(B200_ENODEVICE, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (done[device]) return B200_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
        return fail(B200_ECUDA, "cudaFuncSetAttribute(%s, smem %d): %s", name, smem_bytes, cudaGetErrorString(e));
    done[device] = true;
    return B200_OK;
}

int encode_tmap_2byte(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (g_encode == nullptr) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
                return fail(B200_ECUDA, "cuTensorMapEncodeTiled not available from the driver: %s",
                            cudaGetErrorString(e));
            }
            g_encode = reinterpret_cast<EncodeFn>(fn);
        }
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
        return fail(B200_EINVAL, "tensor base address %p is not 16-byte aligned", base);
    }
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t estrides[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estrides[i] = 1;
        if (i + 1 < rank) {
            if (strides_bytes[i] % 16 != 0) {
                return fail(B200_EINVAL, "stride of dimension %d (%llu bytes) is not a multiple of 16 bytes",
                            i + 1, static_cast<unsigned long long>(strides_bytes[i]));
            }
            gstrides[i] = strides_bytes[i];
        }
    }
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                          const_cast<void*>(base), gdims, gstrides, gbox, estrides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(B200_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dim0 %llu, box0 %u)",
                    static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]), box[0]);
    }
    return B200_OK;
}

}  // namespace b200

extern "C" {

const char* b200_last_error(void) { return b200::t_error; }

const char* b200_version(void) { return "b200dl 0.1 (sm_100a)"; }

int b200_device_status(uint32_t* code) {
    if (code == nullptr) return b200::fail(B200_EINVAL, "code is null");
    const b200::DeviceInfo* dev = b200::current_device();
    if (dev == nullptr) return B200_ENODEVICE;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return b200::fail(B200_ECUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    e = cudaMemcpy(code, dev->status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return b200::fail(B200_ECUDA, "reading the status word: %s", cudaGetErrorString(e));
    if (*code != 0) {
        e = cudaMemset(dev->status, 0, sizeof(uint32_t));
        if (e != cudaSuccess) return b200::fail(B200_ECUDA, "clearing the status word: %s", cudaGetErrorString(e));
    }
    return B200_OK;
}

}  // extern "C"
