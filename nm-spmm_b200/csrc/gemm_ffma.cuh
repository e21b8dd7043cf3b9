// Exact-FP32 vector-wise N:M sparse GEMM for sm_100a: persistent, stream-K scheduled.
//
// Work is measured in units of one k window of one MS x NS tile of C, numbered tile
// by tile.  The units are cut into contiguous ranges, one per CTA:
//   * automatic schedule: as many whole tiles as fill complete waves of resident
//     CTAs, then the units of the remaining tiles in equal ranges, one per resident
//     CTA, so the last wave is as full as the others (no partial last wave);
//   * explicit split_k = S: one range per (tile, K slice), as the reference's
//     gridDim.z slices (src/kernel_64x128_8x8.cu:17-37).
// A CTA walks its range window by window.  Each window's operands are streamed into
// a STAGES-deep shared-memory ring by the TMA engine, completion counted on
// mbarriers: one tiled tensor copy for the window of A, one for the window of B, and
// small bulk copies for the indices.  The ring runs across tile boundaries, so the
// next tile's operands arrive while the current tile is finished and stored.  One
// CTA barrier per window keeps the warps in step and frees the previous window's
// stage, which the warps take turns refilling.  Per window the ring holds
//     As  [KS][MS]   the dense k window of A (A is col-major, so k-row r is MS
//                    contiguous floats): 32 rows; HIGH pairs of windows share one
//                    column_info list and may be staged as one 64-row window
//     Bs  [WS][NS]   the window's compressed rows of B
//     Ds  [..]       the window's packed indices for the vectors of the tile
//     Cs  [..][64]   HIGH only: the window's column_info lists of the index blocks
//                    under the tile; a packed index is a rank into its block's list
// and the gather of the reference (src/kernel_64x128_8x8.cu:139-159) stays what it
// was: the shared-memory row address As[k(p)].  Every warp owns one 32-column
// vector, so that row is warp-uniform; the 8x8 register tile reads two 128-bit words
// of A and two of B per 32 packed two-lane FMAs (64 FMAs).  Unlike the reference's
// high-sparsity kernels the A window is staged dense (one TMA box instead of one
// copy per used column), which frees the CTA tile from the packed index block size.
//
// A range that covers a whole tile stores C directly.  Otherwise the piece goes to
// a scratch slot; the last piece of a tile to arrive (per-tile counter) adds the
// pieces in k order and writes C, so the result does not depend on arrival order.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"

namespace nmspmm {

template <int MS, int NS, int WM, int WS, int KS_, int MODE>
struct FfmaCfg {
    static constexpr int KS = KS_;                       // rows of A staged per window: 32, or 64 (a merged HIGH window)
    static constexpr bool PAIR = (MODE == kModeLow && KS_ == 64);    // LOW staged as pairs of 32-k windows (WS = 2 n_keep)
    static constexpr bool BANDED = (MODE == kModeLow && WS % 16 == 0);   // 16:32 and unpruned: the tile order may be banded (see tile_position)
    static_assert(KS_ == 64 || (MODE == kModeLow && KS_ == 32), "LOW windows are 32 k wide, staged singly or in pairs; HIGH windows are 64 k wide");
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
    static constexpr int BAR_BYTES = 128;                // STAGES mbarriers and two flag words
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 128;   // + alignment slack
    static_assert(MS % WM == 0 && (WM == 64 || WM == 32 || WM == 16), "warp tile");
    static_assert(STAGES * 8 + 8 <= BAR_BYTES, "barrier block");
    static_assert(THREADS <= 512, "tile too large");
};

// MULTI: finished tiles go to every buffer of g.C at (ldc, col0) -- the fused all-gather of a
// column-sharded rank; otherwise to g.C[0] as a private M x N matrix.  A template flag, not a
// run-time one: the kernel sits at the edge of its 128-register budget and the extra
// loop in the epilogue cost the plain form 5-10 % through the register allocation alone.
template <int MS, int NS, int WM, int WS, int KS_, int MODE, bool MULTI>
__device__ __forceinline__ void nm_gemm_ffma_body(const GemmArgs& g, const CUtensorMap& map_a, const CUtensorMap& map_b,
                                                  const GemmOutputs& outs)
{
    using Cfg = FfmaCfg<MS, NS, WM, WS, KS_, MODE>;
    constexpr int KS = Cfg::KS, QT = Cfg::QT, NCW = Cfg::NCW, NCT = Cfg::NCT, MT = Cfg::MT, STAGES = Cfg::STAGES;
    constexpr int E = MT * 2;                              // float4 words of C per thread

    extern __shared__ unsigned char smem_raw[];
    // 128-byte aligned base (dynamic shared memory is only guaranteed 16); everything
    // below is addressed by 32-bit shared addresses.
    const uint32_t ring = (smem_u32(smem_raw) + 127u) & ~127u;
    const uint32_t bars = ring + STAGES * Cfg::STAGE_BYTES;        // full[STAGES]: a stage's operands have landed
    const uint32_t flags = bars + STAGES * 8;                      // abort word, last-piece word
    const uint32_t abort_word = flags, last_word = flags + 4;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        prefetch_tensor_map(&map_a);                       // the first copies would otherwise wait for the descriptors
        prefetch_tensor_map(&map_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bars + s * 8, 1);                    // full: one arrive (with expect_tx) by the filling warp
        }
        sts_volatile_s32(abort_word, 0);
        sts_volatile_s32(last_word, 0);
        mbar_init_fence();
    }
    __syncthreads();
    grid_dependency_wait();                                // everything above overlapped the tail of the kernel ahead

    const int qs_shift = g.qs_shift;                       // log2(vectors per packed index block)
    const int layout_shift = qs_shift + 5;                 // log2(columns per packed index block)
    const int d_chunk = WS << qs_shift;                    // ints of one index block's window
    const uint32_t d_bytes = static_cast<uint32_t>(d_chunk) * 4u;
    const int vec = warp % QT, wm = warp / QT;
    const int lm = (lane & 15) >> 1;

    // This CTA's unit range (one range per CTA: the grid has n_virtual CTAs).
    int u_begin, u_end;
    {
        long long u0, u1;
        virtual_range(g.sched, blockIdx.x, u0, u1);
        u_begin = static_cast<int>(u0);
        u_end = static_cast<int>(u1);
    }

    // Tile number -> position.  The 16:32 and unpruned variants take the banded order of
    // gemm_args.h (the planner bands them when B outgrows L2); with that arithmetic in them
    // they also run 1 - 7 % faster on every one of the reference's 100 benchmark shapes (a
    // different register allocation: these kernels sit at their 128-register limit and the
    // compiler's choices there move the result by several per cent either way).  The other
    // variants were slower with it (12:32 up to 6 %, 8:32 1 %, 4:32 10 % at 4096^3): the
    // planner never bands them and they keep the plain row-by-row expression.
    auto tile_position = [&](int tile, int& ty, int& tx) {
        if constexpr (Cfg::BANDED) {
            tile_coords(tile, g.tiles_x, (g.M + MS - 1) / MS, ty, tx);
        } else {
            ty = tile / g.tiles_x;
            tx = tile - ty * g.tiles_x;
        }
    };

    // ---- filling one stage: the whole warp calls this (warp-uniform arguments) ----
    // Unit `u` goes to stage s, which the caller knows to be free.
    auto fill = [&](int s, int u) {
        const uint32_t full = bars + s * 8;
        const int tile = u / g.sched.n_win, win = u - tile * g.sched.n_win;
        int ty, tx;
        tile_position(tile, ty, tx);
        const int bj = tx * NS, bi = ty * MS;
        const int cols = min(NS, g.N - bj);
        const int lb0 = bj >> layout_shift;                // first packed index block under the tile
        const int nlb = ((bj + cols - 1) >> layout_shift) - lb0 + 1;
        const uint32_t as = ring + s * Cfg::STAGE_BYTES, bs = as + Cfg::A_BYTES, ds = bs + Cfg::B_BYTES;
        if (lane == 0) {
            mbar_arrive_expect_tx(full, Cfg::TX_FIXED + nlb * (d_bytes + (MODE == kModeHigh ? 256u : 0u)));
            tma_load_2d(as, &map_a, bi, win * KS, full);      // rows/columns past the tensor arrive as zeros
            tma_load_2d(bs, &map_b, bj, win * WS, full);
        }
        __syncwarp();
        if (lane < nlb) {
            const int* src = g.D + ((static_cast<size_t>(lb0 + lane) * g.W) << qs_shift) + static_cast<size_t>(win) * d_chunk;
            bulk_g2s(ds + lane * d_bytes, src, d_bytes, full);
            if (MODE == kModeHigh) {
                // one list per merged 64-k window
                const int* ci = g.cinfo + (static_cast<size_t>(lb0 + lane) * g.sched.n_win + win) * 64;
                bulk_g2s(ds + Cfg::D_BYTES + lane * 256, ci, 256, full);
            }
        }
    };

    // Prologue: the first STAGES-1 windows, one filling warp each.  Window number j of the
    // range (unit u_begin + j) always lives in stage j % STAGES.
    for (int j = 0; j < STAGES - 1 && u_begin + j < u_end; ++j)
        if (j % NCW == warp) fill(j, u_begin + j);

    int s = 0, use = 0;                                    // stage of the window being multiplied, and its use count
    bool alive = true;                                     // no wait of this warp has given up yet
    const uint32_t a_rel = (wm * WM + lm * (MT >= 4 ? 4 : 2)) * 4;
    const uint32_t b_rel = Cfg::A_BYTES + (vec * kVecLen + (lane >> 4) * 8 + (lane & 1) * 4) * 4;

    // One iteration per piece: consecutive windows of one tile.
    for (int cu = u_begin; cu < u_end;) {
        const int tile = cu / g.sched.n_win;
        const int piece_n = min((tile + 1) * g.sched.n_win, u_end) - cu;
        uint32_t d_rel, ci_rel;
        bool live;
        {
            int ty, tx;
            tile_position(tile, ty, tx);
            const int bj = tx * NS;
            live = (vec * kVecLen < g.N - bj);             // vectors past N idle but keep the ring moving
            const int q = (bj >> 5) + vec;                 // global vector number
            const int lb = (q >> qs_shift) - (bj >> layout_shift);   // its index block, relative to the tile
            d_rel = Cfg::A_BYTES + Cfg::B_BYTES + (lb * d_chunk + (lane << qs_shift) + (q & ((1 << qs_shift) - 1))) * 4;
            ci_rel = Cfg::A_BYTES + Cfg::B_BYTES + Cfg::D_BYTES + lb * 256;
        }

        float2 acc[MT][4];                                 // row i, column pairs (0,1) (2,3) | (16,17) (18,19)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][c] = make_float2(0.0f, 0.0f);

        for (int w = 0; w < piece_n; ++w) {
            // One CTA barrier per window keeps the warps in step (left alone they drift
            // apart by the whole depth of the ring and then wait for one another); the
            // second CTA of the SM computes meanwhile.  After it the previous window's
            // stage is free: the warps take turns loading the window STAGES-1 ahead into it.
            __syncthreads();
            {
                const int next = cu + w + STAGES - 1;
                // (never re-arm a stage after a wait gave up: its barrier may still be in the
                // phase that did not complete, and a second arrival would underflow its count)
                if (next < u_end && ((cu + w) % NCW) == warp && alive) {
                    if (lane == 0) fence_proxy_async();    // the CTA's reads of the stage come before the TMA's writes
                    __syncwarp();
                    fill(s == 0 ? STAGES - 1 : s - 1, next);
                }
            }
            // A wait that gives up raises the CTA's abort word; every later wait then fails
            // at once, the warps keep walking the loop for the barriers' sake, and the CTA
            // leaves together at the end of the piece without storing anything.
            const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(bars + s * 8, use & 1, abort_word));
            alive = alive && ok;
            if (live && ok) {
                const uint32_t st = ring + s * Cfg::STAGE_BYTES;
                const uint32_t as = st + a_rel, bs = st + b_rel;

                // Lane p resolves the window's p-th index of this warp's vector to a byte
                // offset into As (HIGH: rank -> local column through the block's list); the
                // offsets are handed round the warp by shuffle as the k loop needs them.
                int my_off = 0;
                if (lane < WS) {
                    int k = lds_s32(st + d_rel);
                    if constexpr (MODE == kModeHigh) k = lds_s32(st + ci_rel + k * 4);
                    if constexpr (Cfg::PAIR) k += (lane >= WS / 2) ? 32 : 0;       // second window of the pair
                    my_off = k * (MS * 4);
                }
#define NMSPMM_OFF(p) __shfl_sync(0xffffffffu, my_off, (p))

                float a[2][MT];
                float4 b[2][2];
                auto load = [&](int p, int buf, int off) {
                    const uint32_t ap = as + off;
                    if constexpr (MT == 8) {
                        const float4 lo = lds_f4(ap), hi = lds_f4(ap + 32 * 4);
                        a[buf][0] = lo.x; a[buf][1] = lo.y; a[buf][2] = lo.z; a[buf][3] = lo.w;
                        a[buf][4] = hi.x; a[buf][5] = hi.y; a[buf][6] = hi.z; a[buf][7] = hi.w;
                    } else if constexpr (MT == 4) {
                        const float4 lo = lds_f4(ap);
                        a[buf][0] = lo.x; a[buf][1] = lo.y; a[buf][2] = lo.z; a[buf][3] = lo.w;
                    } else {
                        const float2 lo = lds_f2(ap);
                        a[buf][0] = lo.x; a[buf][1] = lo.y;
                    }
                    const uint32_t bp = bs + p * (NS * 4);
                    b[buf][0] = lds_f4(bp);
                    b[buf][1] = lds_f4(bp + 16 * 4);
                };
                load(0, 0, NMSPMM_OFF(0));
                int off_next = (WS > 1) ? NMSPMM_OFF(1) : 0;
#pragma unroll
                for (int p = 0; p < WS; ++p) {
                    if (p + 1 < WS) {
                        load(p + 1, (p + 1) & 1, off_next);
                        if (p + 2 < WS) off_next = NMSPMM_OFF(p + 2);
                    }
                    // Packed FP32 FMA (two lanes per instruction): the B pairs come straight
                    // out of the 128-bit loads, the A value is duplicated into a pair.  Each
                    // component rounds exactly like a scalar fmaf.
                    const float4 b0 = b[p & 1][0], b1 = b[p & 1][1];
                    const float2 bp0 = make_float2(b0.x, b0.y), bp1 = make_float2(b0.z, b0.w);
                    const float2 bp2 = make_float2(b1.x, b1.y), bp3 = make_float2(b1.z, b1.w);
#pragma unroll
                    for (int i = 0; i < MT; ++i) {
                        const float2 aa = make_float2(a[p & 1][i], a[p & 1][i]);
                        if (i & 1) {                               // serpentine over the column pairs
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
            if (++s == STAGES) { s = 0; ++use; }
        }
        __syncthreads();
        if (cu + piece_n >= u_end) grid_launch_dependents();   // last piece: only stores are left
        if (lds_volatile_s32(abort_word) != 0) {           // a bounded wait gave up somewhere in the CTA
            if (tid == 0) atomicMax(g.status, kDevTimeoutFull);
            break;
        }

        // ---------------------------------------------------------------- end of the piece
        int ty, tx;
        tile_position(tile, ty, tx);
        const int bj = tx * NS, bi = ty * MS;
        const int col0 = bj + vec * kVecLen + (lane >> 4) * 8 + (lane & 1) * 4;      // and col0 + 16
        auto row_of = [&](int i) {
            return bi + wm * WM + ((MT == 8) ? ((i < 4) ? lm * 4 + i : 32 + lm * 4 + (i - 4))
                                             : ((MT == 4) ? lm * 4 + i : lm * 2 + i));
        };
        auto store_tile = [&]() {
            if (!live) return;
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int r = row_of(i);
                if (r < g.M) {
                    if constexpr (MULTI) {
                        const size_t at = static_cast<size_t>(r) * outs.ldc + outs.col0 + col0;
                        for (int o = 0; o < outs.n_out; ++o) {   // every output (peers' copies of C when gathering)
                            float* cp = output_of(g, outs, o) + at;
                            *reinterpret_cast<float4*>(cp) = make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y);
                            *reinterpret_cast<float4*>(cp + 16) = make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y);
                        }
                    } else {
                        float* cp = g.C + static_cast<size_t>(r) * g.N + col0;
                        *reinterpret_cast<float4*>(cp) = make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y);
                        *reinterpret_cast<float4*>(cp + 16) = make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y);
                    }
                }
            }
        };
        if (piece_n == g.sched.n_win) {
            store_tile();                                  // the whole tile was computed here
        } else {
            // A piece of the tile: park it in this range's scratch slot; the last piece to
            // arrive adds all pieces in k order and writes C.
            int v_first, v_last;
            tile_contributors(g.sched, tile, v_first, v_last);
            auto slot_of = [&](int v) -> size_t { return static_cast<size_t>(piece_slot(g.sched, v, tile)); };
            float4* slots = reinterpret_cast<float4*>(g.partial);
            constexpr size_t kSlot = static_cast<size_t>(E) * NCT;             // float4 words per slot
            {
                float4* mine = slots + slot_of(blockIdx.x) * kSlot + tid;
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    __stcg(mine + (2 * i) * NCT, make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y));
                    __stcg(mine + (2 * i + 1) * NCT, make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y));
                }
            }
            if (g.counters == nullptr) {                   // many pieces per tile: the reduction kernel adds them
                cu += piece_n;
                continue;
            }
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned n_pieces = static_cast<unsigned>(v_last - v_first + 1);
                const unsigned prev = atomicAdd(&g.counters[tile], 1u);
                const bool last = (prev == n_pieces - 1u);
                if (last) g.counters[tile] = 0u;               // ready for the next call
                sts_volatile_s32(last_word, last ? 1 : 0);
            }
            __syncthreads();
            const bool last = (lds_volatile_s32(last_word) != 0);
            if (last) {
                __threadfence();
                if (live) {
                    // the accumulators are free again: gather the pieces into them
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[i][c] = make_float2(0.0f, 0.0f);
                    for (int v = v_first; v <= v_last; ++v) {          // fixed order: ascending k
                        const float4* src = slots + slot_of(v) * kSlot + tid;
#pragma unroll
                        for (int i = 0; i < MT; ++i) {
                            const float4 x = __ldcg(src + (2 * i) * NCT), y = __ldcg(src + (2 * i + 1) * NCT);
                            acc[i][0].x += x.x; acc[i][0].y += x.y; acc[i][1].x += x.z; acc[i][1].y += x.w;
                            acc[i][2].x += y.x; acc[i][2].y += y.y; acc[i][3].x += y.z; acc[i][3].y += y.w;
                        }
                    }
                    store_tile();
                }
            }
            __syncthreads();                               // last_flag is reused by the next piece
        }

        cu += piece_n;                                     // on to the next piece of the range
    }
}

// The two kernels: private C (the argument block of old), and C to several buffers.
template <int MS, int NS, int WM, int WS, int KS_, int MODE>
__global__ void __launch_bounds__((FfmaCfg<MS, NS, WM, WS, KS_, MODE>::THREADS), (FfmaCfg<MS, NS, WM, WS, KS_, MODE>::MIN_BLOCKS))
nm_gemm_ffma_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b)
{
    nm_gemm_ffma_body<MS, NS, WM, WS, KS_, MODE, false>(g, map_a, map_b, GemmOutputs {});
}

template <int MS, int NS, int WM, int WS, int KS_, int MODE>
__global__ void __launch_bounds__((FfmaCfg<MS, NS, WM, WS, KS_, MODE>::THREADS), (FfmaCfg<MS, NS, WM, WS, KS_, MODE>::MIN_BLOCKS))
nm_gemm_ffma_multi_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const GemmOutputs outs)
{
    nm_gemm_ffma_body<MS, NS, WM, WS, KS_, MODE, true>(g, map_a, map_b, outs);
}

// Host-side launcher of one variant: encodes the two tensor maps (A as [K][M] with an
// MS x KS box, B as [W][N] with an NS x WS box) and sets the dynamic shared-memory
// limit once per device.
template <int MS, int NS, int WM, int WS, int KS_, int MODE, bool MULTI>
cudaError_t launch_ffma(const GemmArgs& a, const GemmOutputs& outs, int grid, cudaStream_t st)
{
    using Cfg = FfmaCfg<MS, NS, WM, WS, KS_, MODE>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        if (MULTI)
            e = cudaFuncSetAttribute(nm_gemm_ffma_multi_kernel<MS, NS, WM, WS, KS_, MODE>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        else
            e = cudaFuncSetAttribute(nm_gemm_ffma_kernel<MS, NS, WM, WS, KS_, MODE>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    CUtensorMap map_a, map_b;
    e = encode_tensor_map_2d(&map_a, a.A, outs.lda ? outs.lda : a.M, a.sched.n_win * Cfg::KS, MS, Cfg::KS);
    if (e != cudaSuccess) return e;
    // (test hook: a box one row short delivers fewer bytes than the stage's barrier expects,
    // so that the kernel's bounded waits run out; see nmspmm_test_short_fill)
    e = encode_tensor_map_2d(&map_b, a.B, a.N, a.W, NS, WS - (g_test_short_fill ? 1 : 0));
    if (e != cudaSuccess) return e;
    if (MULTI)
        return launch_overlapped(nm_gemm_ffma_multi_kernel<MS, NS, WM, WS, KS_, MODE>, grid, Cfg::THREADS, Cfg::SMEM_BYTES, st,
                                 a, map_a, map_b, outs);
    return launch_overlapped(nm_gemm_ffma_kernel<MS, NS, WM, WS, KS_, MODE>, grid, Cfg::THREADS, Cfg::SMEM_BYTES, st, a, map_a, map_b);
}

#define NMSPMM_FFMA_VARIANT(ID, NKEEP, MS, NS, WM, WS, KS, MODE)                                            \
    FfmaVariant { ID, MS, NS, NKEEP, WS, KS, MODE, FfmaCfg<MS, NS, WM, WS, KS, MODE>::THREADS,               \
                  FfmaCfg<MS, NS, WM, WS, KS, MODE>::SMEM_BYTES, FfmaCfg<MS, NS, WM, WS, KS, MODE>::STAGES,  \
                  FfmaCfg<MS, NS, WM, WS, KS, MODE>::MIN_BLOCKS, &launch_ffma<MS, NS, WM, WS, KS, MODE, false>,     \
                  &launch_ffma<MS, NS, WM, WS, KS, MODE, true> }

// All tiles for one (kept rows per 32-window, B rows per stage, A rows per stage, MODE).
#define NMSPMM_FFMA_TILES(NKEEP, WS, KS, MODE)                            \
    NMSPMM_FFMA_VARIANT(kTile128x128, NKEEP, 128, 128, 64, WS, KS, MODE), \
    NMSPMM_FFMA_VARIANT(kTile64x128, NKEEP, 64, 128, 64, WS, KS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile32x128, NKEEP, 32, 128, 32, WS, KS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile16x128, NKEEP, 16, 128, 16, WS, KS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile128x256, NKEEP, 128, 256, 64, WS, KS, MODE), \
    NMSPMM_FFMA_VARIANT(kTile16x256, NKEEP, 16, 256, 16, WS, KS, MODE),   \
    NMSPMM_FFMA_VARIANT(kTile32x256, NKEEP, 32, 256, 32, WS, KS, MODE)

}  // namespace nmspmm
