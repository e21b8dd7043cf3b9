// Operands kept in 16-bit storage (IEEE half, bfloat16).
//
// Every half and bfloat16 value is a TF32 value (at most 10 mantissa bits, exponent within
// FP32's), so widening loses nothing and the tensor-core path, which drops the low 13
// mantissa bits of its FP32 operands, multiplies widened 16-bit operands exactly; sums are
// FP32 on both paths.  The conversions therefore sit where the data is touched anyway:
// activations are widened by the kernel that transposes them into the multiply's col-major
// layout, weights once when they are compressed, and the result is rounded (to nearest even)
// by one pass over C.  All three are HBM-bound element-wise kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"

namespace nmspmm {

template <typename T> __device__ __forceinline__ float widen(T v);
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Row-major 16-bit activations [M][K] -> FP32 col-major [K][ld], columns M .. ld-1 zero: the
// transposition of transpose_rows_kernel (preprocess.cu) with the widening folded in.
// 2 M K bytes in, 4 ld K out.
template <typename T>
__global__ void __launch_bounds__(256) transpose_rows_16_kernel(const T* __restrict__ in, float* __restrict__ out, int M, int K, int ld)
{
    __shared__ float patch[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int k0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
    for (int j = ty; j < 32; j += 8) {
        const int m = m0 + j, k = k0 + tx;
        patch[j][tx] = (m < M && k < K) ? widen<T>(in[static_cast<size_t>(m) * K + k]) : 0.0f;
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int k = k0 + j, m = m0 + tx;
        if (k < K && m < ld) out[static_cast<size_t>(k) * ld + m] = patch[tx][j];
    }
}

// n floats -> n 16-bit values, four per thread and step (n % 4 == 0, both 8-byte aligned).
template <typename T>
__global__ void __launch_bounds__(256) narrow_kernel(const float4* __restrict__ in, T* __restrict__ out, size_t n4)
{
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float4 v = in[i];
        union { T h[4]; uint2 u; } w;
        w.h[0] = narrow<T>(v.x); w.h[1] = narrow<T>(v.y); w.h[2] = narrow<T>(v.z); w.h[3] = narrow<T>(v.w);
        reinterpret_cast<uint2*>(out)[i] = w.u;
    }
}

// n 16-bit values -> n floats (n % 4 == 0).
template <typename T>
__global__ void __launch_bounds__(256) widen_kernel(const T* __restrict__ in, float4* __restrict__ out, size_t n4)
{
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        union { T h[4]; uint2 u; } w;
        w.u = reinterpret_cast<const uint2*>(in)[i];
        out[i] = make_float4(widen<T>(w.h[0]), widen<T>(w.h[1]), widen<T>(w.h[2]), widen<T>(w.h[3]));
    }
}

static unsigned flat_grid(size_t n4)
{
    const size_t want = (n4 + 255) / 256;
    return static_cast<unsigned>(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));     // grid-stride: a few CTAs per SM
}

cudaError_t launch_transpose_rows_16(int dtype, const void* in, float* out, int M, int K, int ld, cudaStream_t st)
{
    const dim3 grid((K + 31) / 32, (ld + 31) / 32);
    if (dtype == kDtypeF16)
        transpose_rows_16_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(in), out, M, K, ld);
    else if (dtype == kDtypeBF16)
        transpose_rows_16_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), out, M, K, ld);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_narrow(int dtype, const float* in, void* out, size_t n, cudaStream_t st)
{
    if (n == 0) return cudaSuccess;
    if (n % 4 != 0) return cudaErrorInvalidValue;
    if (dtype == kDtypeF16)
        narrow_kernel<__half><<<flat_grid(n / 4), 256, 0, st>>>(reinterpret_cast<const float4*>(in), static_cast<__half*>(out), n / 4);
    else if (dtype == kDtypeBF16)
        narrow_kernel<__nv_bfloat16><<<flat_grid(n / 4), 256, 0, st>>>(reinterpret_cast<const float4*>(in), static_cast<__nv_bfloat16*>(out), n / 4);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_widen(int dtype, const void* in, float* out, size_t n, cudaStream_t st)
{
    if (n == 0) return cudaSuccess;
    if (n % 4 != 0) return cudaErrorInvalidValue;
    if (dtype == kDtypeF16)
        widen_kernel<__half><<<flat_grid(n / 4), 256, 0, st>>>(static_cast<const __half*>(in), reinterpret_cast<float4*>(out), n / 4);
    else if (dtype == kDtypeBF16)
        widen_kernel<__nv_bfloat16><<<flat_grid(n / 4), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), reinterpret_cast<float4*>(out), n / 4);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace nmspmm
