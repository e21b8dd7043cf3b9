// Exact-FP32 vector-wise N:M sparse GEMM for sm_100a.
//
// One CTA computes an MS x NS tile of C over a contiguous range of k windows
// (its split-K slice).  Each window's operands are streamed into a STAGES-deep
// shared-memory ring by the TMA engine, completion counted on mbarriers: one tiled
// tensor copy for the window of A, one for the window of B, and small bulk copies
// for the indices.  The warps take turns issuing a window's copies (a few
// instructions by one warp per window) and otherwise only compute: there is no
// CTA-wide barrier in the main loop.  Per window the ring holds
//     As  [KS][MS]   the dense k window of A (A is col-major, so k-row r is MS
//                    contiguous floats): 32 rows (LOW) or 64 rows (HIGH)
//     Bs  [WS][NS]   the window's compressed rows of B
//     Ds  [..]       the window's packed indices for the vectors of the tile
//     Cs  [..][64]   HIGH only: the window's column_info lists of the index blocks
//                    under the tile; a packed index is a rank into its block's list
// and the gather of the reference (src/kernel_64x128_8x8.cu:139-159) stays what it
// was: the shared-memory row address As[k(p)].  Every warp owns one 32-column
// vector, so that row is warp-uniform, and the 8x8 register tile reads two 128-bit
// words of A and two of B per 64 FFMAs.  Unlike the reference's high-sparsity
// kernels the A window is staged dense (one TMA box instead of one copy per used
// column), which frees the CTA tile from the packed index block size.
//
// split_k > 1: each slice writes its partial tile to scratch; the last slice to
// arrive (per-tile counter) adds the partials in slice order and writes C, so the
// result does not depend on arrival order.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"

namespace nmspmm {

template <int MS, int NS, int WM, int WS, int MODE>
struct FfmaCfg {
    static constexpr int KS = (MODE == kModeLow) ? 32 : 64;
    static constexpr int QT = NS / kVecLen;              // vectors per tile
    static constexpr int WARPS_M = MS / WM;
    static constexpr int NCW = QT * WARPS_M;             // warps (all of them compute)
    static constexpr int NCT = NCW * 32;
    static constexpr int THREADS = NCT;
    static constexpr int MT = WM / 8;                    // rows per thread (8, 4 or 2)
    static constexpr int DQ = (QT > 4) ? QT : 4;         // index ints per compressed row held per stage
    static constexpr int A_BYTES = KS * MS * 4;
    static constexpr int B_BYTES = WS * NS * 4;
    static constexpr int D_BYTES = ((WS * DQ * 4 + 127) / 128) * 128;
    static constexpr int CI_BYTES = (MODE == kModeHigh) ? QT * 64 * 4 : 0;   // one list per index block under the tile
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + D_BYTES + CI_BYTES;
    static constexpr int TX_FIXED = A_BYTES + B_BYTES;   // bytes the two tensor copies always deliver
    // Registers allow 512 threads per SM at 128 registers; shared memory is split to match.
    static constexpr int MIN_BLOCKS = (512 / THREADS) > 4 ? 4 : (512 / THREADS);
    static constexpr int BUDGET = (224 * 1024) / MIN_BLOCKS - 2048;
    static constexpr int ST0 = BUDGET / STAGE_BYTES;
    static constexpr int STAGES = ST0 < 2 ? 2 : (ST0 > 6 ? 6 : ST0);
    static constexpr int BAR_BYTES = 128;                // 2*STAGES mbarriers + flags
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 128;   // + alignment slack
    static_assert(MS % WM == 0 && (WM == 64 || WM == 32 || WM == 16), "warp tile");
    static_assert(2 * STAGES * 8 + 16 <= BAR_BYTES, "barrier block");
    static_assert(THREADS <= 512, "tile too large");
};

template <int MS, int NS, int WM, int WS, int MODE>
__global__ void __launch_bounds__((FfmaCfg<MS, NS, WM, WS, MODE>::THREADS), (FfmaCfg<MS, NS, WM, WS, MODE>::MIN_BLOCKS))
nm_gemm_ffma_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b)
{
    using Cfg = FfmaCfg<MS, NS, WM, WS, MODE>;
    constexpr int KS = Cfg::KS, QT = Cfg::QT, NCW = Cfg::NCW, NCT = Cfg::NCT, MT = Cfg::MT, STAGES = Cfg::STAGES;

    extern __shared__ unsigned char smem_raw[];
    // 128-byte aligned base (dynamic shared memory is only guaranteed 16).
    unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char* ring = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES);
    volatile int* last_flag = abort_flag + 1;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int bj = blockIdx.x * NS;
    const int bi = blockIdx.y * MS;
    const int z = blockIdx.z;

    int win0, nwin;
    slice_range(g.n_win, g.split_k, z, win0, nwin);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);              // full: one arrive (with expect_tx) by the filling warp
            mbar_init(smem_u32(&bars[STAGES + s]), NCW);   // empty: one arrive per warp
        }
        *abort_flag = 0;
        *last_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();

    const int cols_here = min(NS, g.N - bj);               // columns of the tile that exist
    const int layout_ns = g.qs_l * kVecLen;
    const int lb0 = bj / layout_ns;                        // first packed index block under the tile
    const int nlb = (bj + cols_here - 1) / layout_ns - lb0 + 1;
    const int d_chunk = WS * g.qs_l;                       // ints of one block's window

    const int vec = warp % QT, wm = warp / QT;
    const int lm = (lane & 15) >> 1;
    const bool live = (vec * kVecLen < cols_here);         // vectors past N idle but keep the ring moving

    // ---- filling one stage: the whole warp calls this (warp-uniform arguments) ----
    // Window `itl` (relative to the slice) goes to stage itl % STAGES.  Returns false if
    // the bounded wait for the stage's release gave up.
    const uint32_t d_bytes = static_cast<uint32_t>(d_chunk) * 4u;
    const uint32_t tx_bytes = Cfg::TX_FIXED + nlb * (d_bytes + (MODE == kModeHigh ? 256u : 0u));
    auto fill = [&](int itl) -> bool {
        const int s = itl % STAGES;
        const int win = win0 + itl;
        const uint32_t full = smem_u32(&bars[s]);
        if (itl >= STAGES) {
            const bool ok = mbar_wait_bounded(smem_u32(&bars[STAGES + s]), ((itl / STAGES) - 1) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) {            // the whole warp gives up together
                if (lane == 0) atomicMax(g.status, kDevTimeoutEmpty);
                return false;
            }
        }
        const uint32_t as = smem_u32(ring + s * Cfg::STAGE_BYTES), bs = as + Cfg::A_BYTES, ds = bs + Cfg::B_BYTES;
        if (lane == 0) {
            mbar_arrive_expect_tx(full, tx_bytes);
            tma_load_2d(as, &map_a, bi, win * KS, full);      // rows/columns past the tensor arrive as zeros
            tma_load_2d(bs, &map_b, bj, win * WS, full);
        }
        __syncwarp();
        if (lane < nlb) {
            const int* src = g.D + static_cast<size_t>(lb0 + lane) * g.W * g.qs_l + static_cast<size_t>(win) * d_chunk;
            bulk_g2s(ds + lane * d_bytes, src, d_bytes, full);
            if (MODE == kModeHigh) {
                const int* ci = g.cinfo + (static_cast<size_t>(lb0 + lane) * g.n_win + win) * 64;
                bulk_g2s(ds + Cfg::D_BYTES + lane * 256, ci, 256, full);
            }
        }
        return true;
    };

    // Prologue: the first STAGES-1 windows, one filling warp each.
    for (int itl = 0; itl < STAGES - 1 && itl < nwin; ++itl) {
        if (itl % NCW == warp) fill(itl);
    }

    float2 acc[MT][4];                                     // row i, column pairs (0,1) (2,3) | (16,17) (18,19)
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = make_float2(0.0f, 0.0f);

    const int q = bj / kVecLen + vec;                      // global vector number
    const int lb = q / g.qs_l - lb0;                       // index block of this vector, relative to the tile
    const int d_off = (lb * d_chunk + q % g.qs_l) * 4;
    const int d_stride = g.qs_l * 4;
    const int a_off = (wm * WM + lm * (MT >= 4 ? 4 : 2)) * 4;
    const int b_off = (vec * kVecLen + (lane >> 4) * 8 + (lane & 1) * 4) * 4;

    // The warps take turns refilling the ring: at the top of iteration `it`, warp
    // it % NCW loads window it+STAGES-1 into the stage that window it-1 has left, so
    // STAGES-1 windows are in flight while window `it` is multiplied.
    for (int it = 0; it < nwin; ++it) {
        const int s = it % STAGES;
        const int nxt = it + STAGES - 1;
#ifdef NMSPMM_FFMA_WINDOW_SYNC
        __syncthreads();
#endif
        if (nxt < nwin && it % NCW == warp) {
            if (!fill(nxt)) break;
        }
        const bool ok = mbar_wait_bounded(smem_u32(&bars[s]), (it / STAGES) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {                // the whole warp gives up together
            if (lane == 0) atomicMax(g.status, kDevTimeoutFull);
            break;
        }
        if (live) {
            const unsigned char* st = ring + s * Cfg::STAGE_BYTES;
            const unsigned char* as = st + a_off;
            const unsigned char* bs = st + Cfg::A_BYTES + b_off;
            const unsigned char* ds = st + Cfg::A_BYTES + Cfg::B_BYTES + d_off;

            int row_off[WS];
#pragma unroll
            for (int p = 0; p < WS; ++p) row_off[p] = *reinterpret_cast<const int*>(ds + p * d_stride);
            if constexpr (MODE == kModeHigh) {             // rank -> local column through the block's list
                const int* list = reinterpret_cast<const int*>(st + Cfg::A_BYTES + Cfg::B_BYTES + Cfg::D_BYTES) + lb * 64;
#pragma unroll
                for (int p = 0; p < WS; ++p) row_off[p] = list[row_off[p]];
            }
#pragma unroll
            for (int p = 0; p < WS; ++p) row_off[p] *= (MS * 4);

            float a[2][MT];
            float4 b[2][2];
            auto load = [&](int p, int buf) {
                const unsigned char* ap = as + row_off[p];
                if constexpr (MT == 8) {
                    *reinterpret_cast<float4*>(&a[buf][0]) = *reinterpret_cast<const float4*>(ap);
                    *reinterpret_cast<float4*>(&a[buf][4]) = *reinterpret_cast<const float4*>(ap + 32 * 4);
                } else if constexpr (MT == 4) {
                    *reinterpret_cast<float4*>(&a[buf][0]) = *reinterpret_cast<const float4*>(ap);
                } else {
                    *reinterpret_cast<float2*>(&a[buf][0]) = *reinterpret_cast<const float2*>(ap);
                }
                const unsigned char* bp = bs + p * (NS * 4);
                b[buf][0] = *reinterpret_cast<const float4*>(bp);
                b[buf][1] = *reinterpret_cast<const float4*>(bp + 16 * 4);
            };
            load(0, 0);
#pragma unroll
            for (int p = 0; p < WS; ++p) {
                if (p + 1 < WS) load(p + 1, (p + 1) & 1);
                // Packed FP32 FMA (two lanes per instruction): the B pairs come straight
                // out of the 128-bit loads, the A value is duplicated into a pair.  Each
                // component rounds exactly like a scalar fmaf.
                const float4 b0 = b[p & 1][0], b1 = b[p & 1][1];
                const float2 bp0 = make_float2(b0.x, b0.y), bp1 = make_float2(b0.z, b0.w);
                const float2 bp2 = make_float2(b1.x, b1.y), bp3 = make_float2(b1.z, b1.w);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    const float2 aa = make_float2(a[p & 1][i], a[p & 1][i]);
                    if (i & 1) {                                   // serpentine over the column pairs
                        acc[i][3] = __ffma2_rn(aa, bp3, acc[i][3]);
                        acc[i][2] = __ffma2_rn(aa, bp2, acc[i][2]);
                        acc[i][1] = __ffma2_rn(aa, bp1, acc[i][1]);
                        acc[i][0] = __ffma2_rn(aa, bp0, acc[i][0]);
                    } else {
                        acc[i][0] = __ffma2_rn(aa, bp0, acc[i][0]);
                        acc[i][1] = __ffma2_rn(aa, bp1, acc[i][1]);
                        acc[i][2] = __ffma2_rn(aa, bp2, acc[i][2]);
                        acc[i][3] = __ffma2_rn(aa, bp3, acc[i][3]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[STAGES + s]));
    }

    // ---------------------------------------------------------------- epilogue
    const bool aborted = (*abort_flag != 0);
    const int col0 = bj + vec * kVecLen + (lane >> 4) * 8 + (lane & 1) * 4;      // and col0 + 16
    const bool store = live && !aborted;
    auto row_of = [&](int i) {
        return bi + wm * WM + ((MT == 8) ? ((i < 4) ? lm * 4 + i : 32 + lm * 4 + (i - 4))
                                         : ((MT == 4) ? lm * 4 + i : lm * 2 + i));
    };

    if (g.split_k == 1) {
        if (store) {
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int r = row_of(i);
                if (r < g.M) {
                    float* cp = g.C + static_cast<size_t>(r) * g.N + col0;
                    *reinterpret_cast<float4*>(cp) = make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y);
                    *reinterpret_cast<float4*>(cp + 16) = make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y);
                }
            }
        }
        return;
    }

    const size_t tile = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
    constexpr int E = MT * 2;                              // float4 words per thread
    float4* part = reinterpret_cast<float4*>(g.partial) + (tile * g.split_k) * (static_cast<size_t>(E) * NCT);
    if (!aborted) {
        float4* mine = part + static_cast<size_t>(z) * E * NCT + tid;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            __stcg(mine + (2 * i) * NCT, make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y));
            __stcg(mine + (2 * i + 1) * NCT, make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y));
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(&g.counters[tile], 1u);
        if (prev == static_cast<unsigned>(g.split_k) - 1u) {
            *last_flag = 1;
            g.counters[tile] = 0u;                         // ready for the next call
        }
    }
    __syncthreads();
    if (*last_flag == 0) return;
    __threadfence();
    if (!store) return;
    float4 sum[E];
#pragma unroll
    for (int e = 0; e < E; ++e) sum[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < g.split_k; ++s) {                  // fixed order: slice 0, 1, ...
        const float4* src = part + static_cast<size_t>(s) * E * NCT + tid;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float4 v = __ldcg(src + e * NCT);
            sum[e].x += v.x; sum[e].y += v.y; sum[e].z += v.z; sum[e].w += v.w;
        }
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        const int r = row_of(i);
        if (r < g.M) {
            float* cp = g.C + static_cast<size_t>(r) * g.N + col0;
            *reinterpret_cast<float4*>(cp) = sum[2 * i];
            *reinterpret_cast<float4*>(cp + 16) = sum[2 * i + 1];
        }
    }
}

// Host-side launcher of one variant: encodes the two tensor maps (A as [K][M] with an
// MS x KS box, B as [W][N] with an NS x WS box) and sets the dynamic shared-memory
// limit once per device.
template <int MS, int NS, int WM, int WS, int MODE>
cudaError_t launch_ffma(const GemmArgs& a, dim3 grid, cudaStream_t st)
{
    using Cfg = FfmaCfg<MS, NS, WM, WS, MODE>;
    auto kernel = nm_gemm_ffma_kernel<MS, NS, WM, WS, MODE>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    CUtensorMap map_a, map_b;
    e = encode_tensor_map_2d(&map_a, a.A, a.M, a.n_win * Cfg::KS, MS, Cfg::KS);
    if (e != cudaSuccess) return e;
    e = encode_tensor_map_2d(&map_b, a.B, a.N, a.W, NS, WS);
    if (e != cudaSuccess) return e;
    kernel<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(a, map_a, map_b);
    return cudaGetLastError();
}

#define NMSPMM_FFMA_VARIANT(ID, MS, NS, WM, WS, MODE)                                                   \
    FfmaVariant { ID, MS, NS, WS, MODE, FfmaCfg<MS, NS, WM, WS, MODE>::THREADS,                          \
                  FfmaCfg<MS, NS, WM, WS, MODE>::SMEM_BYTES, FfmaCfg<MS, NS, WM, WS, MODE>::STAGES,      \
                  FfmaCfg<MS, NS, WM, WS, MODE>::MIN_BLOCKS, &launch_ffma<MS, NS, WM, WS, MODE> }

// All tiles for one (WS, MODE).
#define NMSPMM_FFMA_TILES(WS, MODE)                          \
    NMSPMM_FFMA_VARIANT(kTile128x128, 128, 128, 64, WS, MODE), \
    NMSPMM_FFMA_VARIANT(kTile64x128, 64, 128, 64, WS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile32x128, 32, 128, 32, WS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile16x128, 16, 128, 16, WS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile128x256, 128, 256, 64, WS, MODE)

}  // namespace nmspmm
