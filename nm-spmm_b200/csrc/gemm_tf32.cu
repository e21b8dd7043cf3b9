// TF32 tensor-core path of the vector-wise N:M sparse GEMM (tcgen05, accumulators in TMEM).
//
// One CTA computes a 128 x NS tile of C (NS / 32 vectors of 32 columns) over all k windows.
// The dense contraction here is per vector: C[128 x 32] += A_gathered[128 x WS] . B[WS x 32],
// and A_gathered differs for every vector, so the gather cannot be expressed by a shared-
// memory descriptor.  It is done on chip instead:
//   warp 0      TMA producer: per window one tiled copy of the dense A window (As[KS][128],
//               unswizzled), one swizzled tiled copy per vector of its WS x 32 block of B
//               (32-byte chunks swizzled within 128-byte rows: the one legal layout of an
//               MN-major TF32 operand), bulk copies of the packed indices and column lists.
//   warps 2-17  sixteen gather warps in two groups that take the windows in turn (one group's
//               waits overlap the other's copying, which keeps shared memory busy); within
//               a group four warps (one per TMEM lane quadrant) work on one vector.  Thread
//               = row of the tile.  Lane p of a warp resolves the vector's
//               p-th index to a row of As; the offsets go round by shuffle; every thread
//               reads its row's WS gathered values from As (conflict-free: consecutive lanes,
//               consecutive words) and stores them as WS TMEM columns with one tcgen05.st
//               per 16: the A operand of WS / 8 MMAs.  All vectors of a window share one
//               A buffer in TMEM and one hand-off; the buffers form a ring.
//   warp 1      one elected thread issues the window's tcgen05.mma kind::tf32 (M128 N32 K8,
//               A from TMEM, B from shared memory, D = the vector's 32 accumulator columns)
//               back to back and commits to the mbarriers that hand the A buffer and the
//               stage back.
//   epilogue    the gather warps read the accumulators (tcgen05.ld) and store C.
// Every wait is bounded; a wait that gives up raises the device status word.
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"
#include "tcgen05.cuh"

namespace nmspmm {

// Diagnostic build (-DNMSPMM_PROFILE_WAITS): the first gather warp and the MMA warp of every
// CTA add up the cycles they spend in each phase.
#ifdef NMSPMM_PROFILE_WAITS
__device__ unsigned long long g_tf32_profile[16];
#define TF_DECL(...) long long __VA_ARGS__
#define TF_T(name) const long long name = clock64()
#define TF_ADD(acc, since) acc += clock64() - (since)
#define TF_OUT(i, v) atomicAdd(&g_tf32_profile[i], (unsigned long long)(v))
#else
#define TF_DECL(...)
#define TF_T(name)
#define TF_ADD(acc, since)
#define TF_OUT(i, v)
#endif

template <int WS, int KS_, int MODE, int QT_>
struct Tf32Cfg {
    static constexpr int MS = 128, QT = QT_, NS = QT * 32;   // QT = 8: one CTA per SM; QT = 4: two
    static constexpr int KS = KS_;
    static constexpr int G = WS / 8;                       // MMAs (K = 8 each) per vector and window
    static_assert(WS % 8 == 0, "kind::tf32 contracts 8 rows per instruction");
    // 12:32 is staged as pairs of 32-k windows (24 kept rows, three MMAs): PAIR.
    static constexpr bool PAIR = (MODE == kModeLow && KS == 64);
    static constexpr int CH = (WS % 16 == 0) ? 16 : 8;     // TMEM columns per tcgen05.st
    static constexpr int NCH = WS / CH;
    static_assert(WS % CH == 0, "whole stores");
    static constexpr int B_BYTES = QT * WS * 128;          // per vector WS rows of 128 bytes, swizzled; multiple of 1024
    static constexpr int A_BYTES = KS * MS * 4;
    static constexpr int D_BYTES = ((WS * (QT > 4 ? QT : 4) * 4 + 127) / 128) * 128;
    static constexpr int CI_BYTES = (MODE == kModeHigh) ? QT * 256 : 0;
    static constexpr int STAGE_BYTES = ((B_BYTES + A_BYTES + D_BYTES + CI_BYTES + 1023) / 1024) * 1024;
    static constexpr int CTAS_PER_SM = (QT == 8) ? 1 : 2;
    static constexpr int ST0 = ((CTAS_PER_SM == 1 ? 216 : 108) * 1024) / STAGE_BYTES;
    static constexpr int STAGES = ST0 >= 4 ? 4 : 2;        // even: a stage always serves the same group of gather warps
    static constexpr int TMEM_COLS = 512 / CTAS_PER_SM;    // each resident CTA allocates its share
    static constexpr int BUF_COLS = QT * WS;               // one A buffer: every vector of one window
    static constexpr int NBUF0 = (TMEM_COLS - NS) / BUF_COLS;
    static constexpr int NBUF = NBUF0 > 4 ? 4 : NBUF0;     // ring of A buffers beside the accumulators
    static_assert(NBUF >= 1, "no room for an A buffer beside the accumulators");
    static constexpr int GATHER_WARPS = 16;
    // Groups of gather warps that take the windows in turn.  A warp's waits on one mbarrier
    // must follow one another phase by phase (a waiter two phases ahead would see the
    // parity it expects too early), so every A buffer and every stage has to stay with one
    // group: two groups only when both ring depths are even.
    static constexpr int GROUPS = (NBUF % 2 == 0 && STAGES % 2 == 0) ? 2 : 1;
    static constexpr int GROUP_WARPS = GATHER_WARPS / GROUPS;
    static constexpr int VSTEP = GROUP_WARPS / 4;          // vectors a group gathers at a time
    static constexpr int VPW = QT / VSTEP;                 // vectors each gather warp carries per window
    static_assert(GROUP_WARPS % 4 == 0 && QT % VSTEP == 0, "four warps (TMEM lane quadrants) per vector");
    static_assert(VPW % GROUPS == 0, "the epilogue shares each warp's vectors out among the groups");
    static constexpr int THREADS = (2 + GATHER_WARPS) * 32;
    static constexpr int NBARS = 2 * STAGES + 2 * NBUF + 1;
    static constexpr int CTRL_BYTES = ((NBARS * 8 + 16 + 127) / 128) * 128;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CTRL_BYTES + 1024;   // + alignment slack
    static constexpr int ACOL0 = NS;                       // first A-buffer column
    static constexpr bool HALF = false;
};

// Whole warp: each thread stores CH (8 or 16) consecutive 32-bit columns of its own lane.
template <int CH>
__device__ __forceinline__ void tmem_st_chunk(uint32_t taddr, const uint32_t (&v)[CH])
{
    if constexpr (CH == 8) {
        tmem_st_x8(taddr, v);
    } else {
        static_assert(CH == 16, "8 or 16 columns per store");
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
              "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
            : "memory");
    }
}

template <int WS, int KS_, int MODE, int QT_>
__global__ void __launch_bounds__((Tf32Cfg<WS, KS_, MODE, QT_>::THREADS), (Tf32Cfg<WS, KS_, MODE, QT_>::CTAS_PER_SM))
nm_gemm_tf32_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmOutputs outs)
{
    using Cfg = Tf32Cfg<WS, KS_, MODE, QT_>;
    constexpr int MS = Cfg::MS, NS = Cfg::NS, QT = Cfg::QT, KS = Cfg::KS, G = Cfg::G, STAGES = Cfg::STAGES, NBUF = Cfg::NBUF;
    constexpr int CH = Cfg::CH, NCH = Cfg::NCH, VPW = Cfg::VPW;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;          // swizzle atoms want 1024-byte alignment
    const uint32_t bars = ring + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + STAGES * 8;
    const uint32_t bar_aready = bar_empty + STAGES * 8, bar_afree = bar_aready + NBUF * 8;
    const uint32_t bar_acc = bar_afree + NBUF * 8;
    const uint32_t tmem_word = bar_acc + 8, abort_word = tmem_word + 4;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // The first n_dp CTAs take one whole tile each.  The remaining tiles (the partial last
    // wave of a large problem, or all tiles of a small one) are cut into split_k K slices,
    // one CTA each: a slice's accumulators go to its scratch slot and the reduction kernel
    // adds the slots.
    const int n_dp = g.sched.n_dp;
    const bool sliced = static_cast<int>(blockIdx.x) >= n_dp;
    const int n_slices = sliced ? g.sched.split_k : 1;
    const int slot = static_cast<int>(blockIdx.x) - n_dp;  // scratch slot of a sliced CTA
    const int tile = sliced ? n_dp + slot / n_slices : static_cast<int>(blockIdx.x);
    const int ty = tile / g.tiles_x, tx = tile - ty * g.tiles_x;
    const int bi = ty * MS, bj = tx * NS;
    int win0, n_win;                                       // this CTA's k windows: win0 .. win0 + n_win - 1
    slice_range(g.sched.n_win, n_slices, sliced ? slot % n_slices : 0, win0, n_win);
    const int live_vecs = min(QT, (g.N - bj) / 32);        // vectors of the tile that exist
    const int qs_shift = g.qs_shift, layout_shift = qs_shift + 5;
    const int d_chunk = WS << qs_shift;
    const uint32_t d_bytes = static_cast<uint32_t>(d_chunk) * 4u;
    const int lb0 = bj >> layout_shift;
    const int nlb = ((bj + live_vecs * 32 - 1) >> layout_shift) - lb0 + 1;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, Cfg::GROUP_WARPS + 1);           // the window's gather warps + the MMA commit
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(bar_aready + b * 8, Cfg::GROUP_WARPS);
            mbar_init(bar_afree + b * 8, 1);                              // the MMA commit
        }
        mbar_init(bar_acc, 1);
        sts_volatile_s32(abort_word, 0);
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_word, Cfg::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = static_cast<uint32_t>(lds_volatile_s32(tmem_word));

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        for (int it = 0; it < n_win; ++it) {
            const int s = it % STAGES;
            if (it >= STAGES) {
                const bool ok = mbar_wait_bounded(bar_empty + s * 8, ((it / STAGES) - 1) & 1, abort_word);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicMax(g.status, kDevTimeoutEmpty);
                    break;
                }
            }
            const uint32_t st = ring + s * Cfg::STAGE_BYTES, full = bar_full + s * 8;
            const uint32_t as = st + Cfg::B_BYTES, ds = as + Cfg::A_BYTES;
            if (elect_one()) {
                mbar_arrive_expect_tx(full, Cfg::A_BYTES + live_vecs * (WS * 128) +
                                                nlb * (d_bytes + (MODE == kModeHigh ? 256u : 0u)));
                for (int b = 0; b < nlb; ++b) {            // the indices first: the gather starts from them
                    const int* src = g.D + ((static_cast<size_t>(lb0 + b) * g.W) << qs_shift) + static_cast<size_t>(win0 + it) * d_chunk;
                    bulk_g2s(ds + b * d_bytes, src, d_bytes, full);
                    if (MODE == kModeHigh) {
                        const int* ci = g.cinfo + (static_cast<size_t>(lb0 + b) * g.sched.n_win + win0 + it) * 64;
                        bulk_g2s(ds + Cfg::D_BYTES + b * 256, ci, 256, full);
                    }
                }
                tma_load_2d(as, &map_a, bi, (win0 + it) * KS, full);
                for (int v = 0; v < live_vecs; ++v) tma_load_2d(st + v * (WS * 128), &map_b, bj + v * 32, (win0 + it) * WS, full);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = umma_idesc_tf32(128, 32);
        bool alive = true;
        TF_DECL(m_full = 0, m_ready = 0, m_issue = 0);
        TF_T(m_start);
        for (int it = 0; it < n_win; ++it) {
            const int s = it % STAGES, b = it % NBUF;
            TF_T(t0);
            bool ok = mbar_wait_bounded(bar_full + s * 8, (it / STAGES) & 1, abort_word);
            TF_ADD(m_full, t0);
            TF_T(t1);
            ok = ok && mbar_spin_bounded(bar_aready + b * 8, (it / NBUF) & 1, abort_word);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            TF_ADD(m_ready, t1);
            TF_T(t2);
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t st = ring + s * Cfg::STAGE_BYTES;
                const uint32_t abuf = tmem_addr(tmem, 0, Cfg::ACOL0 + b * Cfg::BUF_COLS);
                for (int v = 0; v < live_vecs; ++v) {
#pragma unroll
                    for (int gi = 0; gi < G; ++gi)
                        umma_tf32_ts(tmem_addr(tmem, 0, v * 32), abuf + v * WS + gi * 8,
                                     umma_desc_mn_tf32(st + v * (WS * 128) + gi * 1024), idesc, (it | gi) != 0);
                }
                tc_commit(bar_afree + b * 8);              // the A buffer is free once these MMAs have read it
                tc_commit(bar_empty + s * 8);              // and so are the window's B blocks
            }
            __syncwarp();
            TF_ADD(m_issue, t2);
        }
#ifdef NMSPMM_PROFILE_WAITS
        if (lane == 0) { TF_OUT(7, m_full); TF_OUT(8, m_ready); TF_OUT(9, m_issue); TF_OUT(10, clock64() - m_start); }
#endif
        if (!alive && lane == 0) atomicMax(g.status, kDevTimeoutMma);
        if (elect_one()) tc_commit(bar_acc);               // every MMA has completed: accumulators are final
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ gather warps
        const int gw = warp - 2;                           // 0..15
        const int quad = warp & 3;                         // TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;                  // row of the tile this thread carries
        const int grp = gw / Cfg::GROUP_WARPS;             // its windows: grp, grp + GROUPS, ...
        const int v0 = (gw % Cfg::GROUP_WARPS) >> 2;       // its vectors: v0, v0 + VSTEP, ...
        constexpr int VSTEP = Cfg::VSTEP;
        // where lane p finds index p of vector v0 + 4 i within the staged index block
        uint32_t d_rel[VPW], ci_rel[VPW];
#pragma unroll
        for (int i = 0; i < VPW; ++i) {
            const int q = (bj >> 5) + v0 + VSTEP * i;
            const int lb = (q >> qs_shift) - lb0;
            d_rel[i] = static_cast<uint32_t>(lb * d_chunk + (lane << qs_shift) + (q & ((1 << qs_shift) - 1))) * 4u;
            ci_rel[i] = static_cast<uint32_t>(lb * 256);
        }
        bool alive = true;
        TF_DECL(g_full = 0, g_res = 0, g_free = 0, g_move = 0, g_done = 0);
        TF_T(g_start);
        for (int it = grp; it < n_win; it += Cfg::GROUPS) {
            const int s = it % STAGES, b = it % NBUF;
            TF_T(t0);
            bool ok = mbar_wait_bounded(bar_full + s * 8, (it / STAGES) & 1, abort_word);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            TF_ADD(g_full, t0);
            TF_T(t1);
            const uint32_t st = ring + s * Cfg::STAGE_BYTES;
            const uint32_t as = st + Cfg::B_BYTES + row * 4, ds = st + Cfg::B_BYTES + Cfg::A_BYTES, cs = ds + Cfg::D_BYTES;
            // lane p resolves index p of each of the warp's vectors to a byte offset into As
            uint32_t off[VPW];
#pragma unroll
            for (int i = 0; i < VPW; ++i) {
                int k = 0;
                if (lane < WS && v0 + VSTEP * i < live_vecs) {
                    k = lds_s32(ds + d_rel[i]);
                    if (MODE == kModeHigh) k = lds_s32(cs + ci_rel[i] + k * 4);
                    if (Cfg::PAIR && lane >= WS / 2) k += 32;      // second window of the pair
                }
                off[i] = static_cast<uint32_t>(k) * (MS * 4);
            }
            TF_ADD(g_res, t1);
            TF_T(t2);
            if (it >= NBUF) {
                ok = mbar_wait_bounded(bar_afree + b * 8, ((it / NBUF) - 1) & 1, abort_word);
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                tc_fence_after_sync();
            }
            TF_ADD(g_free, t2);
            TF_T(t3);
#pragma unroll
            for (int i = 0; i < VPW; ++i) {
                const int v = v0 + VSTEP * i;
                if (v < live_vecs) {                       // warp-uniform
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        uint32_t a[CH];
#pragma unroll
                        for (int j = 0; j < CH; ++j) a[j] = lds_u32(as + __shfl_sync(0xffffffffu, off[i], c * CH + j));
                        tmem_st_chunk<CH>(tmem_addr(tmem, quad * 32, Cfg::ACOL0 + b * Cfg::BUF_COLS + v * WS + c * CH), a);
                    }
                }
            }
            TF_ADD(g_move, t3);
            TF_T(t4);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_aready + b * 8);
                mbar_arrive(bar_empty + s * 8);            // this warp has finished reading As of the stage
            }
            TF_ADD(g_done, t4);
        }
#ifdef NMSPMM_PROFILE_WAITS
        if (gw == 0 && lane == 0) {
            TF_OUT(0, g_full); TF_OUT(1, g_res); TF_OUT(2, g_free); TF_OUT(3, g_move); TF_OUT(4, g_done);
            TF_OUT(5, clock64() - g_start); TF_OUT(6, 1);
        }
#endif
        // ------------------------------------------------------------------ epilogue
        bool ok = alive && mbar_wait_bounded(bar_acc, 0, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
            const int r = bi + row;
#pragma unroll 1
            for (int i = grp; i < VPW; i += Cfg::GROUPS) {  // the groups share the warp's vectors out
                const int col = (v0 + VSTEP * i) * 32;
                if (col >= live_vecs * 32) break;
                uint32_t v[32];
                tmem_ld_x32(tmem_addr(tmem, quad * 32, col), v);
                tmem_wait_ld();
                if (sliced) {
                    float4* dst = reinterpret_cast<float4*>(g.partial + (static_cast<size_t>(slot) * MS + row) * NS + col);
#pragma unroll
                    for (int x = 0; x < 8; ++x)
                        dst[x] = make_float4(__uint_as_float(v[4 * x]), __uint_as_float(v[4 * x + 1]),
                                             __uint_as_float(v[4 * x + 2]), __uint_as_float(v[4 * x + 3]));
                } else if (r < g.M) {
                    const size_t at = static_cast<size_t>(r) * outs.ldc + outs.col0 + bj + col;
                    for (int o = 0; o < outs.n_out; ++o) {   // every output (peers' copies of C when gathering)
                        float4* dst = reinterpret_cast<float4*>(output_of(g, outs, o) + at);
#pragma unroll
                        for (int x = 0; x < 8; ++x)
                            dst[x] = make_float4(__uint_as_float(v[4 * x]), __uint_as_float(v[4 * x + 1]),
                                                 __uint_as_float(v[4 * x + 2]), __uint_as_float(v[4 * x + 3]));
                    }
                }
            }
        } else if (lane == 0) {
            atomicMax(g.status, kDevTimeoutMma);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::TMEM_COLS);
    }
}

template <int WS, int KS, int MODE, int QT>
static cudaError_t launch_tf32(const GemmArgs& a, const GemmOutputs& outs, int tiles, cudaStream_t st)
{
    using Cfg = Tf32Cfg<WS, KS, MODE, QT>;
    auto kernel = nm_gemm_tf32_kernel<WS, KS, MODE, QT>;
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
    e = encode_tensor_map_2d(&map_a, a.A, a.M, a.sched.n_win * KS, Cfg::MS, KS, 0);
    if (e != cudaSuccess) return e;
    e = encode_tensor_map_2d(&map_b, a.B, a.N, a.W, 32, WS, 1);      // 32-byte chunks swizzled in 128-byte rows
    if (e != cudaSuccess) return e;
    kernel<<<tiles, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(a, map_a, map_b, outs);
    return cudaGetLastError();
}

#define NMSPMM_TF32_VARIANT(NKEEP, WS, KS, MODE, QT)                                                        \
    { NKEEP, WS, KS, MODE, QT * 32, Tf32Cfg<WS, KS, MODE, QT>::SMEM_BYTES, Tf32Cfg<WS, KS, MODE, QT>::STAGES, \
      &launch_tf32<WS, KS, MODE, QT> }

extern const Tf32Variant kTf32Variants[] = {
    NMSPMM_TF32_VARIANT(32, 32, 32, kModeLow, 8),  NMSPMM_TF32_VARIANT(32, 32, 32, kModeLow, 4),
    NMSPMM_TF32_VARIANT(16, 16, 32, kModeLow, 8),  NMSPMM_TF32_VARIANT(16, 16, 32, kModeLow, 4),
    NMSPMM_TF32_VARIANT(12, 24, 64, kModeLow, 8),  NMSPMM_TF32_VARIANT(12, 24, 64, kModeLow, 4),
    NMSPMM_TF32_VARIANT(8, 8, 32, kModeLow, 8),    NMSPMM_TF32_VARIANT(8, 8, 32, kModeLow, 4),
    NMSPMM_TF32_VARIANT(8, 16, 64, kModeHigh, 8),  NMSPMM_TF32_VARIANT(8, 16, 64, kModeHigh, 4),
    NMSPMM_TF32_VARIANT(4, 8, 64, kModeHigh, 8),   NMSPMM_TF32_VARIANT(4, 8, 64, kModeHigh, 4),
};
extern const int kTf32VariantCount = sizeof(kTf32Variants) / sizeof(kTf32Variants[0]);

#ifdef NMSPMM_PROFILE_WAITS
// Diagnostic build only: reads and clears the phase counters.
extern "C" int nmspmm_debug_tf32_profile(unsigned long long* out16)
{
    if (cudaMemcpyFromSymbol(out16, g_tf32_profile, sizeof(unsigned long long) * 16) != cudaSuccess) return 1;
    unsigned long long zero[16] = {};
    return cudaMemcpyToSymbol(g_tf32_profile, zero, sizeof(zero)) == cudaSuccess ? 0 : 1;
}
#endif

}  // namespace nmspmm
