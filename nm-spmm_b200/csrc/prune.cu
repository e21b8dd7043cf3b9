// Vector-wise N:M magnitude pruning on the GPU: dense weight [K][N] -> compressed values
// BT [W][N] and window-local indices DT [W][Q], the inputs of the index packing and the
// multiply, so that a weight matrix never has to visit the host.
//
// Rule (the package's host generator formats.prune_magnitude states the same): in every
// window of 32 consecutive k rows and for every vector of vec_len (32 or 64) columns keep the
// n_keep rows with the largest sum of squares over the vector's columns, ties to the lower
// row; kept rows in ascending order.  The sum of squares is taken in double precision with
// eight interleaved partial sums combined pairwise -- the order numpy's float64 sum uses for
// a contiguous run of 32 or 64 values -- so the selection is bit-identical to the host's.
//
// One warp per (window, vector); lane = row of the window.  A lane reads its row's
// vec_len floats (whole 128-byte lines), ranks its score against the other 31 by shuffle,
// and the kept lanes write their rows out again.  HBM-bound: K*N*4 bytes in, W*N*4 out.
#include <cuda_runtime.h>
#include <stdint.h>

#include "nmspmm_b200.h"

namespace nmspmm {

template <int VEC>
__global__ void __launch_bounds__(256) prune_magnitude_kernel(const float* __restrict__ dense, float* __restrict__ BT,
                                                             int* __restrict__ DT, int n_windows, int N, int n_keep)
{
    constexpr int V4 = VEC / 4;
    const int lane = threadIdx.x & 31;
    const int nvec = N / VEC;
    const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= static_cast<long long>(n_windows) * nvec) return;      // whole warps leave together
    const int win = static_cast<int>(unit / nvec), v = static_cast<int>(unit - static_cast<long long>(win) * nvec);
    const float4* src = reinterpret_cast<const float4*>(dense + (static_cast<size_t>(win) * 32 + lane) * N + static_cast<size_t>(v) * VEC);
    float4 x[V4];
#pragma unroll
    for (int i = 0; i < V4; ++i) x[i] = __ldg(src + i);
    // eight partial sums over elements j % 8, combined pairwise
    double r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = 0.0;
#pragma unroll
    for (int i = 0; i < V4; ++i) {
        const int b = (i & 1) * 4;
        r[b + 0] += static_cast<double>(x[i].x) * static_cast<double>(x[i].x);
        r[b + 1] += static_cast<double>(x[i].y) * static_cast<double>(x[i].y);
        r[b + 2] += static_cast<double>(x[i].z) * static_cast<double>(x[i].z);
        r[b + 3] += static_cast<double>(x[i].w) * static_cast<double>(x[i].w);
    }
    const double score = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
    // rank among the window's 32 rows: rows with a larger score, or the same score and a lower row, come first
    int rank = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const double other = __shfl_sync(0xffffffffu, score, j);
        rank += (other > score || (other == score && j < lane)) ? 1 : 0;
    }
    const bool keep = rank < n_keep;
    const unsigned kept = __ballot_sync(0xffffffffu, keep);
    if (keep) {
        const int pos = __popc(kept & ((1u << lane) - 1u));            // ascending row order
        const size_t w = static_cast<size_t>(win) * n_keep + pos;
        float4* dst = reinterpret_cast<float4*>(BT + w * N + static_cast<size_t>(v) * VEC);
#pragma unroll
        for (int i = 0; i < V4; ++i) dst[i] = x[i];
        int* d = DT + w * (N / 32) + static_cast<size_t>(v) * (VEC / 32);
#pragma unroll
        for (int h = 0; h < VEC / 32; ++h) d[h] = lane;                 // one index per 32 columns (V = 64: the same twice)
    }
}

}  // namespace nmspmm

extern "C" int nmspmm_prune_device(const float* dense_dev, float* BT_dev, int* DT_dev, int K, int N, int n_keep, int vec_len,
                                   void* stream)
{
    if (!dense_dev || !BT_dev || !DT_dev) return NMSPMM_INVALID_ARGUMENT;
    if (K <= 0 || N <= 0 || K % 32 != 0 || (vec_len != 32 && vec_len != 64) || N % vec_len != 0) return NMSPMM_INVALID_ARGUMENT;
    if (n_keep < 1 || n_keep > 32) return NMSPMM_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(dense_dev) | reinterpret_cast<uintptr_t>(BT_dev)) & 15u) return NMSPMM_INVALID_ARGUMENT;
    const long long units = static_cast<long long>(K / 32) * (N / vec_len);
    const long long blocks = (units + 7) / 8;
    if (blocks >= (1LL << 31)) return NMSPMM_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec_len == 32)
        nmspmm::prune_magnitude_kernel<32><<<static_cast<unsigned>(blocks), 256, 0, st>>>(dense_dev, BT_dev, DT_dev, K / 32, N, n_keep);
    else
        nmspmm::prune_magnitude_kernel<64><<<static_cast<unsigned>(blocks), 256, 0, st>>>(dense_dev, BT_dev, DT_dev, K / 32, N, n_keep);
    return cudaGetLastError() == cudaSuccess ? NMSPMM_OK : NMSPMM_CUDA_ERROR;
}
