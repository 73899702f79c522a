// Self-test of the bounded-wait machinery: a kernel whose consumer waits for bytes that
// never arrive, with a wait limit of milliseconds instead of the kernels' 2 s.  It shows on a
// live GPU what a pipeline bug would look like to a caller: the wait gives up, the site
// code lands in the device status word, every role leaves its loop, the kernel returns and
// the context stays usable.  Nothing here faults, traps or spins without a limit.
#include "ptx_sm100.cuh"
#include "runtime.h"

namespace b200 {
namespace {

constexpr uint32_t kSelftestSite = 0x7e57u;

__global__ void __launch_bounds__(64, 1) wait_expiry_kernel(unsigned long long limit_ns, uint32_t* status) {
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t abort_word;
    const uint32_t full = smem_u32(&bars[0]);    // producer -> consumer
    const uint32_t empty = smem_u32(&bars[1]);   // consumer -> producer
    const WaitGuard guard{&abort_word, status};
    if (threadIdx.x == 0) {
        mbar_init(full, 1);
        mbar_init(empty, 1);
        abort_word = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0 && lane == 0) {
        // Producer: announces 128 bytes for the stage and copies none of them, so the phase
        // can never complete.  It then waits for the consumer's release like a real producer
        // would, and leaves when the consumer's expired wait raises the abort flag.
        mbar_arrive_expect_tx(full, 128);
        (void)mbar_wait_limit(guard, empty, 0, kSelftestSite + 1, 4 * limit_ns);
    } else if (warp == 1) {
        // Consumer: the wait that runs out.
        const bool ok = __all_sync(0xffffffffu, mbar_wait_limit(guard, full, 0, kSelftestSite, limit_ns));
        if (ok && lane == 0) mbar_arrive(empty);
    }
    __syncthreads();
}

}  // namespace
}  // namespace b200

extern "C" int b200_selftest_wait_expiry(uint32_t limit_ms, void* stream) {
    using namespace b200;
    if (limit_ms == 0 || limit_ms > 1000) return fail(B200_EINVAL, "limit_ms must be 1..1000 (got %u)", limit_ms);
    const DeviceInfo* dev = current_device();
    if (dev == nullptr) return B200_ENODEVICE;
    wait_expiry_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<unsigned long long>(limit_ms) * 1000000ull, dev->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200_ECUDA, "launch of the wait self-test failed: %s", cudaGetErrorString(e));
    return B200_OK;
}
