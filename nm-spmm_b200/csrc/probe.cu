// Register-only FFMA loop: measures the FP32 SIMT rate the exact path is bounded by.
#include "common.cuh"
#include "kernels.h"

namespace nmspmm {

constexpr int kProbeIters = 2048;
constexpr int kProbeChains = 16;

__global__ void __launch_bounds__(512) ffma_peak_kernel(float* sink, float x, float y)
{
    float acc[kProbeChains];
#pragma unroll
    for (int c = 0; c < kProbeChains; ++c) acc[c] = x * static_cast<float>(threadIdx.x + c);
    for (int it = 0; it < kProbeIters; ++it) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int c = 0; c < kProbeChains; ++c) acc[c] = fmaf(acc[c], y, x);
    }
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < kProbeChains; ++c) s += acc[c];
    if (s == 123.456f) *sink = s;       // never true in practice; keeps the loop alive
}

// The same loop with the packed two-lane FMA of sm_100.
__global__ void __launch_bounds__(512) ffma2_peak_kernel(float* sink, float x, float y)
{
    float2 acc[kProbeChains / 2];
#pragma unroll
    for (int c = 0; c < kProbeChains / 2; ++c) acc[c] = make_float2(x * (threadIdx.x + c), x * (threadIdx.x - c));
    const float2 yy = make_float2(y, y), xx = make_float2(x, x);
    for (int it = 0; it < kProbeIters; ++it) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int c = 0; c < kProbeChains / 2; ++c) acc[c] = __ffma2_rn(acc[c], yy, xx);
    }
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < kProbeChains / 2; ++c) s += acc[c].x + acc[c].y;
    if (s == 123.456f) *sink = s;
}

cudaError_t measure_ffma_peak(double* tflops, int packed, cudaStream_t st)
{
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    float* sink = nullptr;
    e = cudaMalloc(&sink, sizeof(float));
    if (e != cudaSuccess) return e;
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    const int blocks = sms * 4, threads = 512;
    double best = 0.0;
    for (int rep = 0; rep < 6; ++rep) {
        cudaEventRecord(t0, st);
        if (packed)
            ffma2_peak_kernel<<<blocks, threads, 0, st>>>(sink, 0.999f, 1.0001f);
        else
            ffma_peak_kernel<<<blocks, threads, 0, st>>>(sink, 0.999f, 1.0001f);
        cudaEventRecord(t1, st);
        e = cudaEventSynchronize(t1);
        if (e != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, t0, t1);
        const double flops = 2.0 * blocks * threads * static_cast<double>(kProbeIters) * 8 * kProbeChains;
        if (rep >= 2 && ms > 0.f) best = fmax(best, flops / (ms * 1e-3) / 1e12);
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    cudaFree(sink);
    if (e == cudaSuccess) e = cudaGetLastError();
    *tflops = best;
    return e;
}

}  // namespace nmspmm
