// Measured issue-rate peaks of the device the march kernels are compared with: fp32 FMA and ex2.approx
// throughput with every SM busy on independent register chains.  The march kernels are bound by
// instruction issue, not by memory, so these (not the HBM rate) are the ceilings that explain them.
#include <cuda_runtime.h>

#include "../../include/rgx.h"
#include "rgx_internal.cuh"

namespace {

constexpr int kChains = 8;        // independent dependency chains per thread
constexpr int kThreads = 256;
constexpr int kBlocksPerSm = 8;   // 2048 threads per SM: every scheduler always has a ready warp

__global__ void __launch_bounds__(kThreads) fma_chain_kernel(float x, float y, int iters, float* sink) {
    float a[kChains];
#pragma unroll
    for (int k = 0; k < kChains; ++k) a[k] = (float)(threadIdx.x + k) * 1e-3f;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int k = 0; k < kChains; ++k) a[k] = fmaf(a[k], x, y);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kChains; ++k) s += a[k];
    if (s == 123456.789f) *sink = s;      // never true for the arguments used; keeps the chains alive
}

__global__ void __launch_bounds__(kThreads) ex2_chain_kernel(int iters, float* sink) {
    float a[kChains];
#pragma unroll
    for (int k = 0; k < kChains; ++k) a[k] = (float)(threadIdx.x + k) * 1e-3f;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int k = 0; k < kChains; ++k) {
                float r;
                asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(-a[k]));   // stays within [0.5, 1]
                a[k] = r;
            }
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kChains; ++k) s += a[k];
    if (s == 123456.789f) *sink = s;
}

}  // namespace

extern "C" int rgx_measure_peaks(int device, float* fma_tflops, float* ex2_gops) {
    if (!fma_tflops || !ex2_gops) return RGX_E_INVALID;
    *fma_tflops = 0.f;
    *ex2_gops = 0.f;
    int count = 0, sms = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return RGX_E_CUDA;
    rgx::DeviceGuard guard(device);
    if (!guard.ok ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        return RGX_E_CUDA;
    float* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t s = nullptr;
    int rc = RGX_E_CUDA;
    if (cudaMalloc((void**)&sink, sizeof(float)) == cudaSuccess && cudaEventCreate(&e0) == cudaSuccess &&
        cudaEventCreate(&e1) == cudaSuccess && cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess) {
        const int grid = sms * kBlocksPerSm;
        const double threads = (double)grid * kThreads;
        const int fma_iters = 4096, ex2_iters = 1024;       // a few milliseconds each
        float ms_fma = 0.f, ms_ex2 = 0.f;
        bool ok = true;
        for (int rep = 0; rep < 2 && ok; ++rep) {           // the first repetition warms up
            cudaEventRecord(e0, s);
            rgx::note_launch(), fma_chain_kernel<<<grid, kThreads, 0, s>>>(0.999f, 1e-4f, fma_iters, sink);
            cudaEventRecord(e1, s);
            ok = cudaStreamSynchronize(s) == cudaSuccess && cudaEventElapsedTime(&ms_fma, e0, e1) == cudaSuccess;
        }
        for (int rep = 0; rep < 2 && ok; ++rep) {
            cudaEventRecord(e0, s);
            rgx::note_launch(), ex2_chain_kernel<<<grid, kThreads, 0, s>>>(ex2_iters, sink);
            cudaEventRecord(e1, s);
            ok = cudaStreamSynchronize(s) == cudaSuccess && cudaEventElapsedTime(&ms_ex2, e0, e1) == cudaSuccess;
        }
        if (ok && ms_fma > 0.f && ms_ex2 > 0.f) {
            *fma_tflops = (float)(2.0 * kChains * 4.0 * fma_iters * threads / (ms_fma * 1e-3) / 1e12);
            *ex2_gops = (float)((double)kChains * 4.0 * ex2_iters * threads / (ms_ex2 * 1e-3) / 1e9);
            rc = RGX_OK;
        }
    }
    (void)cudaGetLastError();
    if (s) cudaStreamDestroy(s);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (sink) cudaFree(sink);
    return rc;
}
