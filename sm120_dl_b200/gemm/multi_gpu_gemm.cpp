// test_gemm_multi_gpu: the BF16 GEMM split by N-column blocks over the GPUs of one box, in C++.
//
//   test_gemm_multi_gpu [--gpus G] [--iterations I] [M N K]
//
// One process, one host thread per device (the reference is single-GPU: both of its launchers
// query device 0, gemm/gemm_cute.hpp:343-346; this driver is new).  A is replicated, device d
// holds rows [n0, n1) of B (a contiguous slab of the row-major [N,K] matrix) and a full-width
// C.  Three variants are timed with CUDA events on every device (5 warm-up + I launches, the
// harness protocol of gemm/test.cpp:27-28; the job time is the maximum over devices):
//
//   compute      every device writes its column slab into its own C (ldc = N)
//   fused        b200_gemm_bf16_tn_scatter: the epilogue stores every finished tile into ALL
//                devices' C through peer-mapped pointers (TMA stores over NVLink), so the full
//                C lands on every device without a collective
//   nccl         slab -> ncclAllGather into [G][M][N/G] staging -> one kernel that interleaves
//                the slabs into the row-major C (column slabs are not contiguous)
//
// Without a shape it runs the three M = 16384 shapes of the multi-GPU benchmark configuration.
// The gathered C of device 0 is checked against cuBLAS on device 0 (the reference's
// comparison rule |d| <= 1e-2 + 5e-2 |ref|, gemm/test.cpp:165-230) on a band of rows.
// Exit code 0 = every shape passed.
#include <algorithm>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include "b200dl.h"

namespace {

using bf16 = __nv_bfloat16;
constexpr int kWarmup = 5;
constexpr int kMaxGpus = 8;

struct Shape {
    int M, N, K;
};

// Reusable barrier for the device threads.
class Barrier {
public:
    explicit Barrier(int n) : n_(n) {}
    void wait() {
        std::unique_lock<std::mutex> lock(m_);
        const int gen = gen_;
        if (++count_ == n_) {
            count_ = 0;
            ++gen_;
            cv_.notify_all();
        } else {
            cv_.wait(lock, [&] { return gen != gen_; });
        }
    }

private:
    std::mutex m_;
    std::condition_variable cv_;
    int n_, count_ = 0, gen_ = 0;
};

#define CHECK_CUDA(call)                                                                              \
    do {                                                                                              \
        cudaError_t err_ = (call);                                                                    \
        if (err_ != cudaSuccess) {                                                                    \
            std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(err_), __FILE__, __LINE__); \
            std::exit(2);                                                                             \
        }                                                                                             \
    } while (0)
#define CHECK_NCCL(call)                                                                              \
    do {                                                                                              \
        ncclResult_t err_ = (call);                                                                   \
        if (err_ != ncclSuccess) {                                                                    \
            std::fprintf(stderr, "NCCL error %s at %s:%d\n", ncclGetErrorString(err_), __FILE__, __LINE__); \
            std::exit(2);                                                                             \
        }                                                                                             \
    } while (0)
#define CHECK_B200(call)                                                                   \
    do {                                                                                   \
        if ((call) != B200_OK) {                                                           \
            std::fprintf(stderr, "b200dl error: %s (%s:%d)\n", b200_last_error(), __FILE__, __LINE__); \
            std::exit(2);                                                                  \
        }                                                                                  \
    } while (0)

// staging [G][M][W] -> C [M][G*W]: 16 bytes per thread.
__global__ void interleave_slabs(const uint4* __restrict__ staging, uint4* __restrict__ c, int M, int G, int w16) {
    const long total = static_cast<long>(M) * G * w16;
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
        const int x = static_cast<int>(i % w16);
        const long r = i / w16;
        const int g = static_cast<int>(r % G);
        const long m = r / G;
        c[i] = staging[(static_cast<long>(g) * M + m) * w16 + x];
    }
}

struct DeviceState {
    bf16 *A = nullptr, *B = nullptr, *C = nullptr, *slab = nullptr, *staging = nullptr;
    cudaStream_t stream = nullptr;
    ncclComm_t comm = nullptr;
    float compute_ms = 0.f, fused_ms = 0.f, nccl_ms = 0.f;
};

template <typename Fn>
float timed(cudaStream_t stream, int iterations, Barrier& bar, Fn fn) {
    for (int i = 0; i < kWarmup; ++i) fn();
    CHECK_CUDA(cudaStreamSynchronize(stream));
    bar.wait();
    cudaEvent_t start, stop;
    CHECK_CUDA(cudaEventCreate(&start));
    CHECK_CUDA(cudaEventCreate(&stop));
    CHECK_CUDA(cudaEventRecord(start, stream));
    for (int i = 0; i < iterations; ++i) fn();
    CHECK_CUDA(cudaEventRecord(stop, stream));
    CHECK_CUDA(cudaEventSynchronize(stop));
    float ms = 0.f;
    CHECK_CUDA(cudaEventElapsedTime(&ms, start, stop));
    CHECK_CUDA(cudaEventDestroy(start));
    CHECK_CUDA(cudaEventDestroy(stop));
    bar.wait();
    return ms / iterations;
}

bool run_shape(const Shape& s, int G, int iterations, ncclComm_t* comms) {
    const int M = s.M, N = s.N, K = s.K;
    if (N % (G * 256) != 0) {
        std::fprintf(stderr, "N=%d is not a multiple of 256 x %d GPUs\n", N, G);
        return false;
    }
    const int W = N / G;
    std::vector<bf16> hA(static_cast<size_t>(M) * K), hB(static_cast<size_t>(N) * K);
    std::mt19937 rng(4);
    std::normal_distribution<float> dist(0.f, 1.f / std::sqrt(static_cast<float>(K)));
    for (auto& v : hA) v = __float2bfloat16(dist(rng));
    for (auto& v : hB) v = __float2bfloat16(dist(rng));

    std::vector<DeviceState> dev(G);
    Barrier bar(G);
    int config = -1;
    std::vector<std::thread> threads;
    for (int d = 0; d < G; ++d) {
        threads.emplace_back([&, d] {
            CHECK_CUDA(cudaSetDevice(d));
            DeviceState& me = dev[d];
            me.comm = comms[d];
            CHECK_CUDA(cudaStreamCreateWithFlags(&me.stream, cudaStreamNonBlocking));
            CHECK_CUDA(cudaMalloc(&me.A, hA.size() * sizeof(bf16)));
            CHECK_CUDA(cudaMalloc(&me.B, static_cast<size_t>(W) * K * sizeof(bf16)));
            CHECK_CUDA(cudaMalloc(&me.C, static_cast<size_t>(M) * N * sizeof(bf16)));
            CHECK_CUDA(cudaMalloc(&me.slab, static_cast<size_t>(M) * W * sizeof(bf16)));
            CHECK_CUDA(cudaMalloc(&me.staging, static_cast<size_t>(M) * N * sizeof(bf16)));
            CHECK_CUDA(cudaMemcpy(me.A, hA.data(), hA.size() * sizeof(bf16), cudaMemcpyHostToDevice));
            CHECK_CUDA(cudaMemcpy(me.B, hB.data() + static_cast<size_t>(d) * W * K, static_cast<size_t>(W) * K * sizeof(bf16),
                                  cudaMemcpyHostToDevice));
            CHECK_CUDA(cudaMemset(me.C, 0xff, static_cast<size_t>(M) * N * sizeof(bf16)));   // NaN pattern
            if (d == 0) config = b200_gemm_default_config(M, W, K);
            bar.wait();

            const int n0 = d * W;
            // compute only: own slab into own full-width C
            me.compute_ms = timed(me.stream, iterations, bar, [&] {
                CHECK_B200(b200_gemm_bf16_tn(config, M, W, K, me.A, K, me.B, K, me.C + n0, N, me.stream));
            });
            // fused gather: every device's C, own copy first
            void* dst[kMaxGpus];
            for (int i = 0; i < G; ++i) dst[i] = dev[(d + i) % G].C + n0;
            me.fused_ms = timed(me.stream, iterations, bar, [&] {
                CHECK_B200(b200_gemm_bf16_tn_scatter(config, M, W, K, me.A, K, me.B, K, dst, G, N, me.stream));
            });
            CHECK_CUDA(cudaStreamSynchronize(me.stream));
            bar.wait();
        });
    }
    for (auto& t : threads) t.join();
    threads.clear();

    // Check device 0's gathered C (left by the fused variant) against cuBLAS on a band of rows.
    bool pass = true;
    {
        CHECK_CUDA(cudaSetDevice(0));
        const int rows = std::min(M, 512);
        bf16 *dB = nullptr, *dRef = nullptr;
        CHECK_CUDA(cudaMalloc(&dB, hB.size() * sizeof(bf16)));
        CHECK_CUDA(cudaMalloc(&dRef, static_cast<size_t>(rows) * N * sizeof(bf16)));
        CHECK_CUDA(cudaMemcpy(dB, hB.data(), hB.size() * sizeof(bf16), cudaMemcpyHostToDevice));
        cublasHandle_t handle;
        if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return false;
        const float alpha = 1.f, beta = 0.f;
        // row-major C[rows,N] = A[rows,K] B[N,K]^T  ==  column-major C^T[N,rows] = B(T) A
        cublasStatus_t st = cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, N, rows, K, &alpha, dB, CUDA_R_16BF, K, dev[0].A,
                                         CUDA_R_16BF, K, &beta, dRef, CUDA_R_16BF, N, CUBLAS_COMPUTE_32F,
                                         CUBLAS_GEMM_DEFAULT_TENSOR_OP);
        CHECK_CUDA(cudaDeviceSynchronize());
        std::vector<bf16> got(static_cast<size_t>(rows) * N), ref(got.size());
        CHECK_CUDA(cudaMemcpy(got.data(), dev[0].C, got.size() * sizeof(bf16), cudaMemcpyDeviceToHost));
        CHECK_CUDA(cudaMemcpy(ref.data(), dRef, ref.size() * sizeof(bf16), cudaMemcpyDeviceToHost));
        size_t bad = 0;
        for (size_t i = 0; i < got.size(); ++i) {
            const float g = __bfloat162float(got[i]), r = __bfloat162float(ref[i]);
            if (!(std::fabs(g - r) <= 1.0e-2f + 5.0e-2f * std::fabs(r))) ++bad;
        }
        pass = st == CUBLAS_STATUS_SUCCESS && bad == 0;
        if (!pass) std::fprintf(stderr, "gathered C differs from cuBLAS in %zu of %zu elements\n", bad, got.size());
        cublasDestroy(handle);
        cudaFree(dB);
        cudaFree(dRef);
    }

    // NCCL variant (timed after the check so that the check sees the fused result)
    for (int d = 0; d < G; ++d) {
        threads.emplace_back([&, d] {
            CHECK_CUDA(cudaSetDevice(d));
            DeviceState& me = dev[d];
            me.nccl_ms = timed(me.stream, iterations, bar, [&] {
                CHECK_B200(b200_gemm_bf16_tn(config, M, W, K, me.A, K, me.B, K, me.slab, W, me.stream));
                CHECK_NCCL(ncclAllGather(me.slab, me.staging, static_cast<size_t>(M) * W, ncclBfloat16, me.comm, me.stream));
                interleave_slabs<<<1184, 256, 0, me.stream>>>(reinterpret_cast<const uint4*>(me.staging),
                                                               reinterpret_cast<uint4*>(me.C), M, G, W / 8);
            });
            CHECK_CUDA(cudaStreamSynchronize(me.stream));
            uint32_t code = 0;
            CHECK_B200(b200_device_status(&code));
            if (code != 0) {
                std::fprintf(stderr, "device %d: a kernel gave up a bounded wait (status 0x%x)\n", d, code);
                std::exit(3);
            }
            cudaFree(me.A);
            cudaFree(me.B);
            cudaFree(me.C);
            cudaFree(me.slab);
            cudaFree(me.staging);
            cudaStreamDestroy(me.stream);
        });
    }
    for (auto& t : threads) t.join();

    float compute = 0.f, fused = 0.f, nccl = 0.f;
    for (const auto& d : dev) {
        compute = std::max(compute, d.compute_ms);
        fused = std::max(fused, d.fused_ms);
        nccl = std::max(nccl, d.nccl_ms);
    }
    const double flops = 2.0 * M * N * K;
    const b200_gemm_config* cfg = b200_gemm_get_config(config);
    std::printf("multi_gpu M=%d N=%d K=%d gpus=%d config=%s compute_ms=%.4f tflops=%.1f fused_gather_ms=%.4f tflops_fused=%.1f "
                "nccl_gather_ms=%.4f tflops_nccl=%.1f verify=%s\n",
                M, N, K, G, cfg ? cfg->name : "?", compute, flops / compute / 1e9, fused, flops / fused / 1e9, nccl,
                flops / nccl / 1e9, pass ? "PASS" : "FAIL");
    return pass;
}

}  // namespace

int main(int argc, char** argv) {
    int gpus = 0, iterations = 20;
    std::vector<Shape> shapes;
    std::vector<int> positional;
    for (int i = 1; i < argc; ++i) {
        if (std::strcmp(argv[i], "--gpus") == 0 && i + 1 < argc) {
            gpus = std::atoi(argv[++i]);
        } else if (std::strcmp(argv[i], "--iterations") == 0 && i + 1 < argc) {
            iterations = std::atoi(argv[++i]);
        } else if (argv[i][0] != '-') {
            positional.push_back(std::atoi(argv[i]));
        } else {
            std::fprintf(stderr, "usage: %s [--gpus G] [--iterations I] [M N K]\n", argv[0]);
            return 1;
        }
    }
    if (positional.size() == 3) {
        shapes.push_back({positional[0], positional[1], positional[2]});
    } else if (positional.empty()) {
        shapes = {{16384, 4096, 4096}, {16384, 14336, 4096}, {16384, 4096, 14336}};
    } else {
        std::fprintf(stderr, "usage: %s [--gpus G] [--iterations I] [M N K]\n", argv[0]);
        return 1;
    }
    int available = 0;
    CHECK_CUDA(cudaGetDeviceCount(&available));
    if (gpus <= 0) gpus = available;
    if (gpus > available || gpus > kMaxGpus || gpus < 1 || iterations < 1) {
        std::fprintf(stderr, "need 1..%d GPUs (have %d) and a positive iteration count\n", kMaxGpus, available);
        return 1;
    }
    // every device maps every other device's memory
    for (int d = 0; d < gpus; ++d) {
        CHECK_CUDA(cudaSetDevice(d));
        for (int p = 0; p < gpus; ++p) {
            if (p == d) continue;
            int can = 0;
            CHECK_CUDA(cudaDeviceCanAccessPeer(&can, d, p));
            if (!can) {
                std::fprintf(stderr, "device %d cannot map device %d's memory\n", d, p);
                return 1;
            }
            cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) CHECK_CUDA(e);
            (void)cudaGetLastError();
        }
    }
    ncclComm_t comms[kMaxGpus];
    int devs[kMaxGpus];
    for (int d = 0; d < gpus; ++d) devs[d] = d;
    CHECK_NCCL(ncclCommInitAll(comms, gpus, devs));
    bool ok = true;
    for (const Shape& s : shapes) ok = run_shape(s, gpus, iterations, comms) && ok;
    for (int d = 0; d < gpus; ++d) ncclCommDestroy(comms[d]);
    return ok ? 0 : 1;
}
