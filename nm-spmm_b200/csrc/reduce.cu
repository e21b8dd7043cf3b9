// Parallel reduction of tile pieces (split-K with many slices per tile).
//
// The multiply parks a piece of a tile -- its accumulators, in the thread-fragment order
// of the kernel that produced them -- in a scratch slot.  With few pieces per tile the
// last piece to arrive adds them up inside the multiply itself.  With many (deep K, few
// tiles) that serial walk by one CTA would outlast the multiply, so the pieces are left
// in scratch and this kernel adds them: one CTA per (tile, fragment row, half row), every
// thread summing one float4 word over the tile's pieces in ascending k order.  The
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

constexpr int kReduceInFlight = 16;   // loads of one thread that are issued before the first is added

// CTAS_PER_ROW = 2: one CTA per (tile, fragment row, one of the row's two float4 words), for
// tiles of many pieces (deep K): the pieces number in the tens and every round of loads costs a
// trip to L2, so sixteen loads are in flight before the first is added.  CTAS_PER_ROW = 1: a
// CTA adds both words, four loads of each in flight -- fewer, fuller CTAs for the common
// case of a handful of pieces, where the launch is what costs.
template <int MS, int NS, int WM, int CTAS_PER_ROW>
__global__ void __launch_bounds__((FragmentMap<MS, NS, WM>::NCT))
nm_reduce_pieces_kernel(const GemmArgs g, const GemmOutputs outs, int first_tile)
{
    using Map = FragmentMap<MS, NS, WM>;
    constexpr int NCT = Map::NCT, MT = Map::MT;
    constexpr int WORDS = 2 / CTAS_PER_ROW, FLIGHT = (CTAS_PER_ROW == 2) ? kReduceInFlight : 4;
    constexpr size_t kSlot = static_cast<size_t>(2 * MT) * NCT;       // float4 words per slot
    const int half = (CTAS_PER_ROW == 2) ? (blockIdx.x & 1) : 0;
    const int i = (blockIdx.x / CTAS_PER_ROW) % MT, tile = first_tile + (blockIdx.x / CTAS_PER_ROW) / MT;
    const int tid = threadIdx.x;
    wait_for_the_multiply();
    if (*reinterpret_cast<volatile int*>(g.status) != 0) return;      // a wait of the multiply gave up: the pieces are incomplete, leave C alone
    int v_first, v_last;
    tile_contributors(g.sched, tile, v_first, v_last);
    if (v_first == v_last) return;                         // one range held the whole tile and stored it
    int ty, tx;
    tile_coords(tile, g.tiles_x, (g.M + MS - 1) / MS, ty, tx);
    const int bj = tx * NS, bi = ty * MS;
    const int r = bi + Map::row(tid, i), c = bj + Map::col0(tid) + 16 * half;
    if (Map::vec(tid) * kVecLen >= g.N - bj || r >= g.M) return;       // vectors past N, rows past M
    const float4* slots = reinterpret_cast<const float4*>(g.partial) + (2 * i + half) * NCT + tid;
    // Slot of range v's piece (piece_slot): one per range with an explicit split; with the
    // automatic schedule two per range, the second for a tile the range entered part-way
    // through its own course -- which only the tile's first contributor can have done.
    const long long slot_first = piece_slot(g.sched, v_first, tile);
    const bool explicit_split = g.sched.split_k > 0;
    const int n_dp = g.sched.n_dp;
    float4 sum[WORDS];
#pragma unroll
    for (int w = 0; w < WORDS; ++w) sum[w] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int v = v_first; v <= v_last; v += FLIGHT) {
        float4 x[FLIGHT][WORDS];
#pragma unroll
        for (int u = 0; u < FLIGHT; ++u) {
            if (v + u <= v_last) {
                const long long slot = (v + u == v_first) ? slot_first : (explicit_split ? v + u : 2LL * (v + u - n_dp));
#pragma unroll
                for (int w = 0; w < WORDS; ++w) x[u][w] = __ldcg(slots + static_cast<size_t>(slot) * kSlot + w * NCT);
            }
        }
#pragma unroll
        for (int u = 0; u < FLIGHT; ++u) {
            if (v + u <= v_last) {
#pragma unroll
                for (int w = 0; w < WORDS; ++w) {
                    sum[w].x += x[u][w].x; sum[w].y += x[u][w].y; sum[w].z += x[u][w].z; sum[w].w += x[u][w].w;
                }
            }
        }
    }
    const size_t at = static_cast<size_t>(r) * outs.ldc + outs.col0 + c;
    for (int o = 0; o < outs.n_out; ++o) {
        float* cp = output_of(g, outs, o) + at;
#pragma unroll
        for (int w = 0; w < WORDS; ++w) *reinterpret_cast<float4*>(cp + 16 * w) = sum[w];
    }
}

template <int MS, int NS, int WM>
static cudaError_t launch_reduce(const GemmArgs& a, const GemmOutputs& outs, int first_tile, int n_tiles, cudaStream_t st)
{
    using Map = FragmentMap<MS, NS, WM>;
    // pieces per tile, about: the ranges that are not whole tiles over the tiles they cover
    const int pieces = a.sched.split_k > 0 ? a.sched.split_k : (a.sched.n_virtual - a.sched.n_dp) / (n_tiles > 0 ? n_tiles : 1) + 1;
    if (pieces > kReduceInFlight / 2)
        return launch_after_multiply(nm_reduce_pieces_kernel<MS, NS, WM, 2>, n_tiles * Map::MT * 2, Map::NCT, st, a, outs, first_tile);
    return launch_after_multiply(nm_reduce_pieces_kernel<MS, NS, WM, 1>, n_tiles * Map::MT, Map::NCT, st, a, outs, first_tile);
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
// ((tile - first_tile) * split_k + z) holds a slice's 128 x NS accumulator tile row-major.
// A thread adds EPT float4 words of a tile, one after the other, over its slices in ascending k
// order, and writes those whose row and columns of C exist.  EPT = 1 with sixteen loads in
// flight for tiles of many slices (deep K: every round of loads is a trip to L2); EPT = 4 with
// four in flight otherwise (fewer CTAs of fewer registers, more of which are resident before
// the multiply ends: the launch is what costs there).
template <int NS, int EPT, int MS = 128>
__global__ void __launch_bounds__(256) nm_reduce_slices_kernel(const GemmArgs g, const GemmOutputs outs, int first_tile)
{
    constexpr int V4 = NS / 4;                             // float4 words per tile row; MS = rows of a slot
    constexpr int FLIGHT = (EPT == 1) ? kReduceInFlight : 4;   // loads in flight per thread
    constexpr int CTAS = MS * V4 / (256 * EPT);            // per tile
    static_assert(CTAS >= 1 && CTAS * 256 * EPT == MS * V4, "whole CTAs per tile");
    const int sliced_tile = blockIdx.x / CTAS, e0 = (blockIdx.x % CTAS) * (256 * EPT) + threadIdx.x;
    const int tile = first_tile + sliced_tile;
    int ty, tx;
    tile_coords(tile, g.tiles_x, (g.M + MS - 1) / MS, ty, tx);
    const int bi = ty * MS, bj = tx * NS;
    const int S = g.sched.split_k;
    wait_for_the_multiply();
    if (*reinterpret_cast<volatile int*>(g.status) != 0) return;      // a wait of the multiply gave up: the slices are incomplete, leave C alone
#pragma unroll 1
    for (int q = 0; q < EPT; ++q) {
        const int e = e0 + q * 256;
        const int row = e / V4, c4 = e % V4;
        if (bi + row >= g.M || bj + c4 * 4 >= g.N) continue;
        const float4* src = reinterpret_cast<const float4*>(g.partial) + static_cast<size_t>(sliced_tile) * S * (MS * V4) + e;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < S; z += FLIGHT) {
            float4 x[FLIGHT];
#pragma unroll
            for (int u = 0; u < FLIGHT; ++u)
                if (z + u < S) x[u] = __ldcg(src + static_cast<size_t>(z + u) * (MS * V4));
#pragma unroll
            for (int u = 0; u < FLIGHT; ++u)
                if (z + u < S) { sum.x += x[u].x; sum.y += x[u].y; sum.z += x[u].z; sum.w += x[u].w; }
        }
        const size_t at = static_cast<size_t>(bi + row) * outs.ldc + outs.col0 + bj + c4 * 4;
        for (int o = 0; o < outs.n_out; ++o) *reinterpret_cast<float4*>(output_of(g, outs, o) + at) = sum;
    }
}

cudaError_t launch_reduce_slices(int ns, const GemmArgs& a, const GemmOutputs& outs, int first_tile, int n_tiles, cudaStream_t st, int ms)
{
    if (n_tiles <= 0) return cudaSuccess;
    const bool many = a.sched.split_k > kReduceInFlight / 2;
    if (ns == 256 && ms == 128)
        return many ? launch_after_multiply(nm_reduce_slices_kernel<256, 1>, n_tiles * 32, 256, st, a, outs, first_tile)
                    : launch_after_multiply(nm_reduce_slices_kernel<256, 4>, n_tiles * 8, 256, st, a, outs, first_tile);
    if (ns == 128 && ms == 128)
        return many ? launch_after_multiply(nm_reduce_slices_kernel<128, 1>, n_tiles * 16, 256, st, a, outs, first_tile)
                    : launch_after_multiply(nm_reduce_slices_kernel<128, 4>, n_tiles * 4, 256, st, a, outs, first_tile);
    // the few-row tiles of gemm_tf32_skinny.cu: slots of ms x 128
    if (ns == 128 && ms == 64) return launch_after_multiply(nm_reduce_slices_kernel<128, 1, 64>, n_tiles * 8, 256, st, a, outs, first_tile);
    if (ns == 128 && ms == 32) return launch_after_multiply(nm_reduce_slices_kernel<128, 1, 32>, n_tiles * 4, 256, st, a, outs, first_tile);
    if (ns == 128 && ms == 16) return launch_after_multiply(nm_reduce_slices_kernel<128, 1, 16>, n_tiles * 2, 256, st, a, outs, first_tile);
    return cudaErrorInvalidValue;
}

}  // namespace nmspmm
