// Parallel reduction of tile pieces (split-K with many slices per tile).
//
// The multiply parks a piece of a tile -- its accumulators, in the thread-fragment order
// of the kernel that produced them -- in a scratch slot.  With few pieces per tile the
// last piece to arrive adds them up inside the multiply itself.  With many (deep K, few
// tiles) that serial walk by one CTA would outlast the multiply, so the pieces are left
// in scratch and this kernel adds them: one CTA per (tile, fragment row), every thread
// summing its own two float4 words over the tile's pieces in ascending k order.  The
// order is fixed, so the result is the same from run to run and the same as the in-kernel
// reduction's.
#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"

namespace nmspmm {

// The reduction kernels are launched with programmatic stream serialisation: the launch is
// set up while the multiply still runs and the grid starts as soon as the multiply's last
// CTA has exited, instead of a launch latency later (these launches follow multiplies that
// last 15-100 us).  This wait is what orders the reads below after the multiply's writes.
__device__ __forceinline__ void wait_for_the_multiply() { grid_dependency_wait(); }

template <typename... KArgs, typename... Args>
static cudaError_t launch_after_multiply(void (*kernel)(KArgs...), unsigned blocks, unsigned threads, cudaStream_t st, Args... args)
{
    return launch_overlapped(kernel, blocks, threads, 0, st, args...);
}

// Thread-fragment map of the FFMA kernels' accumulators for a tile MS x NS with warp tile
// WM x 32: thread tid holds rows row(i), i < MT, and columns col0 .. col0 + 3 and
// col0 + 16 .. col0 + 19 of them; the slot stores fragment row i as float4 words
// (2 i) * NCT + tid and (2 i + 1) * NCT + tid.
template <int MS, int NS, int WM>
struct FragmentMap {
    static constexpr int QT = NS / kVecLen;
    static constexpr int NCT = QT * (MS / WM) * 32;
    static constexpr int MT = WM / 8;
    __device__ static int vec(int tid) { return (tid >> 5) % QT; }
    __device__ static int col0(int tid) { return vec(tid) * kVecLen + ((tid & 31) >> 4) * 8 + (tid & 1) * 4; }
    __device__ static int row(int tid, int i)
    {
        const int wm = (tid >> 5) / QT, lm = (tid & 15) >> 1;
        return wm * WM + ((MT == 8) ? ((i < 4) ? lm * 4 + i : 32 + lm * 4 + (i - 4)) : ((MT == 4) ? lm * 4 + i : lm * 2 + i));
    }
};

template <int MS, int NS, int WM>
__global__ void __launch_bounds__((FragmentMap<MS, NS, WM>::NCT))
nm_reduce_pieces_kernel(const GemmArgs g, const GemmOutputs outs, int first_tile)
{
    using Map = FragmentMap<MS, NS, WM>;
    constexpr int NCT = Map::NCT, MT = Map::MT;
    constexpr size_t kSlot = static_cast<size_t>(2 * MT) * NCT;       // float4 words per slot
    const int tile = first_tile + blockIdx.x / MT, i = blockIdx.x % MT;
    const int tid = threadIdx.x;
    wait_for_the_multiply();
    if (*reinterpret_cast<volatile int*>(g.status) != 0) return;      // a wait of the multiply gave up: the pieces are incomplete, leave C alone
    int v_first, v_last;
    tile_contributors(g.sched, tile, v_first, v_last);
    if (v_first == v_last) return;                         // one range held the whole tile and stored it
    const int ty = tile / g.tiles_x, tx = tile - ty * g.tiles_x;
    const int bj = tx * NS, bi = ty * MS;
    const int r = bi + Map::row(tid, i), c = bj + Map::col0(tid);
    if (Map::vec(tid) * kVecLen >= g.N - bj || r >= g.M) return;       // vectors past N, rows past M
    const float4* slots = reinterpret_cast<const float4*>(g.partial);
    float4 sx = make_float4(0.f, 0.f, 0.f, 0.f), sy = sx;
    for (int v = v_first; v <= v_last; v += 4) {
        float4 x[4], y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (v + u <= v_last) {
                const float4* src = slots + static_cast<size_t>(piece_slot(g.sched, v + u, tile)) * kSlot + tid;
                x[u] = __ldcg(src + (2 * i) * NCT);
                y[u] = __ldcg(src + (2 * i + 1) * NCT);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (v + u <= v_last) {
                sx.x += x[u].x; sx.y += x[u].y; sx.z += x[u].z; sx.w += x[u].w;
                sy.x += y[u].x; sy.y += y[u].y; sy.z += y[u].z; sy.w += y[u].w;
            }
        }
    }
    const size_t at = static_cast<size_t>(r) * outs.ldc + outs.col0 + c;
    for (int o = 0; o < outs.n_out; ++o) {
        float* cp = output_of(g, outs, o) + at;
        *reinterpret_cast<float4*>(cp) = sx;
        *reinterpret_cast<float4*>(cp + 16) = sy;
    }
}

template <int MS, int NS, int WM>
static cudaError_t launch_reduce(const GemmArgs& a, const GemmOutputs& outs, int first_tile, int n_tiles, cudaStream_t st)
{
    using Map = FragmentMap<MS, NS, WM>;
    return launch_after_multiply(nm_reduce_pieces_kernel<MS, NS, WM>, n_tiles * Map::MT, Map::NCT, st, a, outs, first_tile);
}

cudaError_t launch_reduce_pieces(int tile_id, const GemmArgs& a, const GemmOutputs& outs, int first_tile, int n_tiles, cudaStream_t st)
{
    if (n_tiles <= 0) return cudaSuccess;
    switch (tile_id) {
    case kTile128x128: return launch_reduce<128, 128, 64>(a, outs, first_tile, n_tiles, st);
    case kTile64x128: return launch_reduce<64, 128, 64>(a, outs, first_tile, n_tiles, st);
    case kTile32x128: return launch_reduce<32, 128, 32>(a, outs, first_tile, n_tiles, st);
    case kTile16x128: return launch_reduce<16, 128, 16>(a, outs, first_tile, n_tiles, st);
    case kTile128x256: return launch_reduce<128, 256, 64>(a, outs, first_tile, n_tiles, st);
    case kTile16x256: return launch_reduce<16, 256, 16>(a, outs, first_tile, n_tiles, st);
    case kTile32x256: return launch_reduce<32, 256, 32>(a, outs, first_tile, n_tiles, st);
    default: return cudaErrorInvalidValue;
    }
}

// The tensor-core path's K slices: the tiles from first_tile on are sliced; slot
// ((tile - first_tile) * split_k + z) holds a slice's 128 x NS accumulator tile row-major.  One CTA adds the slices of 16 rows of a tile, in ascending
// k order, and writes the rows and columns of C that exist.
template <int NS>
__global__ void __launch_bounds__(256) nm_reduce_slices_kernel(const GemmArgs g, const GemmOutputs outs, int first_tile)
{
    constexpr int MS = 128, ROWS = 16, V4 = NS / 4;        // float4 words per tile row
    const int sliced_tile = blockIdx.x / (MS / ROWS), r0 = (blockIdx.x % (MS / ROWS)) * ROWS;
    const int tile = first_tile + sliced_tile;
    const int ty = tile / g.tiles_x, tx = tile - ty * g.tiles_x;
    const int bi = ty * MS, bj = tx * NS;
    const int S = g.sched.split_k;
    wait_for_the_multiply();
    if (*reinterpret_cast<volatile int*>(g.status) != 0) return;      // a wait of the multiply gave up: the slices are incomplete, leave C alone
    const float4* slots = reinterpret_cast<const float4*>(g.partial) + static_cast<size_t>(sliced_tile) * S * (MS * V4);
    for (int e = threadIdx.x; e < ROWS * V4; e += 256) {
        const int row = r0 + e / V4, c4 = e % V4;
        if (bi + row >= g.M || bj + c4 * 4 >= g.N) continue;
        const float4* src = slots + static_cast<size_t>(row) * V4 + c4;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < S; z += 4) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (z + u < S) x[u] = __ldcg(src + static_cast<size_t>(z + u) * (MS * V4));
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (z + u < S) { sum.x += x[u].x; sum.y += x[u].y; sum.z += x[u].z; sum.w += x[u].w; }
        }
        const size_t at = static_cast<size_t>(bi + row) * outs.ldc + outs.col0 + bj + c4 * 4;
        for (int o = 0; o < outs.n_out; ++o) *reinterpret_cast<float4*>(output_of(g, outs, o) + at) = sum;
    }
}

cudaError_t launch_reduce_slices(int ns, const GemmArgs& a, const GemmOutputs& outs, int first_tile, int n_tiles, cudaStream_t st)
{
    const int blocks = n_tiles * (128 / 16);
    if (blocks <= 0) return cudaSuccess;
    if (ns == 256) return launch_after_multiply(nm_reduce_slices_kernel<256>, blocks, 256, st, a, outs, first_tile);
    if (ns == 128) return launch_after_multiply(nm_reduce_slices_kernel<128>, blocks, 256, st, a, outs, first_tile);
    return cudaErrorInvalidValue;
}

}  // namespace nmspmm
