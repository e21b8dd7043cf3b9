// Index packing on the GPU: bit-exact device versions of the reference's host
// loops (src/preprocessing.cu of the reference).  Integer, HBM-bound work: every
// global access is coalesced, staged through shared memory where the layout
// change would otherwise scatter.
#include "common.cuh"
#include "kernels.h"

namespace nmspmm {

// transIndex (src/preprocessing.cu:3-15): rows of every odd pruning window get
// +pruning_M.  Element-wise, in place.
__global__ void trans_index_kernel(int* __restrict__ DT, long long total, int Q, int pruning_N, int pruning_M)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int w = static_cast<int>(e / Q);
        if ((w / pruning_N) & 1) DT[e] += pruning_M;
    }
}

// PreProcessing_low_sparsity (src/preprocessing.cu:80-100): [W][Q] -> [Q/Qs][W][Qs].
// A CTA moves a 32-row x 32-int patch: rows are read coalesced along q, transposed
// in shared memory, and written as runs of 32*Qs consecutive ints per index block.
__global__ void __launch_bounds__(256) retile_kernel(const int* __restrict__ DT, int* __restrict__ D, int W, int Q, int Qs)
{
    __shared__ int patch[32][33];
    const int q0 = blockIdx.x * 32, w0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int w = w0 + r, q = q0 + tx;
        if (w < W && q < Q) patch[r][tx] = DT[static_cast<size_t>(w) * Q + q];
    }
    __syncthreads();
    const int run = 32 * Qs;                       // ints one index block contributes from this patch
    for (int t = threadIdx.x; t < 1024; t += 256) {
        const int qb = t / run, rem = t % run;
        const int r = rem / Qs, qs = rem % Qs;
        const int w = w0 + r, q = q0 + qb * Qs + qs;
        if (w < W && q < Q)
            D[static_cast<size_t>(q / Qs) * W * Qs + static_cast<size_t>(w) * Qs + qs] = patch[r][qb * Qs + qs];
    }
}

// PreProcessing_high_sparsity (src/preprocessing.cu:17-78), optionally with
// transIndex folded in.  A CTA handles one merged window (pn rows) of up to 32
// index blocks: the window's rows are read coalesced into shared memory, then each
// warp takes blocks in turn: it ORs a 64-bit mask of the local columns its block
// uses, writes the ascending list (-1 padded) to column_info and each index's rank
// (population count of the mask below it) to the re-tiled D.
//   pn, pm: merged window (rows kept / width, pm <= 64).  fuse != 0: DT holds raw
//   0..pm/2-1 indices and rows x >= pn/2 of a window belong to its odd half.
constexpr int kHighBlocksPerCta = 32;
__global__ void __launch_bounds__(256) preprocess_high_kernel(const int* __restrict__ DT, int* __restrict__ D,
                                                              int* __restrict__ cinfo, int pm, int pn, int W, int Q,
                                                              int Qs, int fuse)
{
    extern __shared__ int rows[];                  // [pn][kHighBlocksPerCta * Qs + Qs]: padded, see pitch
    const int win = blockIdx.x;
    const int blk0 = blockIdx.y * kHighBlocksPerCta;
    const int nblk_total = Q / Qs;
    const int nblk = min(kHighBlocksPerCta, nblk_total - blk0);
    const int width = nblk * Qs;                   // ints per row held here
    // a warp reads one block's [pn][Qs] indices, Qs from each row: Qs extra ints per row
    // put consecutive rows Qs banks apart (an unpadded pitch made that an 8-way conflict)
    const int pitch = kHighBlocksPerCta * Qs + Qs;
    for (int t = threadIdx.x; t < pn * width; t += blockDim.x) {
        const int x = t / width, c = t % width;
        int v = DT[static_cast<size_t>(win * pn + x) * Q + blk0 * Qs + c];
        if (fuse && x >= pn / 2) v += pm / 2;
        rows[x * pitch + c] = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwin = W / pn;
    const int per = pn * Qs;                       // indices of one (block, window)
    for (int b = warp; b < nblk; b += 8) {
        unsigned lo = 0u, hi = 0u;
        for (int e = lane; e < per; e += 32) {
            const int v = rows[(e / Qs) * pitch + b * Qs + e % Qs] & 63;
            if (v < 32) lo |= 1u << v; else hi |= 1u << (v - 32);
        }
        lo = __reduce_or_sync(0xffffffffu, lo);
        hi = __reduce_or_sync(0xffffffffu, hi);
        const unsigned long long mask = (static_cast<unsigned long long>(hi) << 32) | lo;
        const int used = __popcll(mask);
        const size_t blk = blk0 + b;
        int* ci = cinfo + (blk * nwin + win) * pm;
        for (int x = lane; x < pm; x += 32) {
            if ((mask >> x) & 1ull) ci[__popcll(mask & ((1ull << x) - 1ull))] = x;
            if (x >= used) ci[x] = -1;
        }
        int* out = D + blk * W * Qs + static_cast<size_t>(win) * per;      // [pn][Qs] run of this window
        for (int e = lane; e < per; e += 32) {
            const int v = rows[(e / Qs) * pitch + b * Qs + e % Qs] & 63;
            out[e] = __popcll(mask & ((1ull << v) - 1ull));
        }
    }
}

__global__ void fill_kernel(int* p, int n, int value)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = value;
}

cudaError_t launch_trans_index(int* DT, int W, int Q, int pruning_N, int pruning_M, cudaStream_t st)
{
    const long long total = static_cast<long long>(W) * Q;
    if (total == 0) return cudaSuccess;
    const long long want = (total + 255) / 256;
    const int blocks = static_cast<int>(want < 148LL * 16 ? want : 148LL * 16);
    trans_index_kernel<<<blocks, 256, 0, st>>>(DT, total, Q, pruning_N, pruning_M);
    return cudaGetLastError();
}

cudaError_t launch_retile(const int* DT, int* D, int W, int Q, int Qs, cudaStream_t st)
{
    if (W == 0 || Q == 0) return cudaSuccess;
    dim3 grid((Q + 31) / 32, (W + 31) / 32);
    retile_kernel<<<grid, 256, 0, st>>>(DT, D, W, Q, Qs);
    return cudaGetLastError();
}

cudaError_t launch_preprocess_high(const int* DT, int* D, int* cinfo, int pm, int pn, int W, int Q, int Qs,
                                   int fuse, int tail_ints, cudaStream_t st)
{
    if (W == 0 || Q == 0) return cudaSuccess;
    const int nblk = Q / Qs, nwin = W / pn;
    dim3 grid(nwin, (nblk + kHighBlocksPerCta - 1) / kHighBlocksPerCta);
    const size_t smem = static_cast<size_t>(pn) * (kHighBlocksPerCta * Qs + Qs) * sizeof(int);
    preprocess_high_kernel<<<grid, 256, smem, st>>>(DT, D, cinfo, pm, pn, W, Q, Qs, fuse);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (tail_ints > 0) {
        fill_kernel<<<(tail_ints + 255) / 256, 256, 0, st>>>(cinfo + static_cast<size_t>(nblk) * nwin * pm, tail_ints, -1);
        e = cudaGetLastError();
    }
    return e;
}

// Row-major activations [M][K] -> the reference's col-major A, i.e. [K][ld] with ld >= M,
// columns M .. ld-1 zero.  32 x 32 patches through padded shared memory: reads coalesced
// along k, writes coalesced along m.  HBM-bound: 4 M K bytes in, 4 ld K out.
__global__ void __launch_bounds__(256) transpose_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int M, int K, int ld)
{
    __shared__ float patch[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int k0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
    for (int j = ty; j < 32; j += 8) {
        const int m = m0 + j, k = k0 + tx;
        patch[j][tx] = (m < M && k < K) ? in[static_cast<size_t>(m) * K + k] : 0.0f;
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int k = k0 + j, m = m0 + tx;
        if (k < K && m < ld) out[static_cast<size_t>(k) * ld + m] = patch[tx][j];
    }
}

cudaError_t launch_transpose_rows(const float* in, float* out, int M, int K, int ld, cudaStream_t st)
{
    const dim3 grid((K + 31) / 32, (ld + 31) / 32);
    transpose_rows_kernel<<<grid, 256, 0, st>>>(in, out, M, K, ld);
    return cudaGetLastError();
}

}  // namespace nmspmm
