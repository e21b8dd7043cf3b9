// TF32 tensor-core path of the vector-wise N:M sparse GEMM (tcgen05, accumulators in TMEM).
//
// One CTA computes a 128 x 256 tile of C (eight 32-column vectors) over all k windows.
// The dense contraction here is per vector: C[128 x 32] += A_gathered[128 x WS] . B[WS x 32],
// and A_gathered differs for every vector, so the gather cannot be expressed by a shared-
// memory descriptor.  It is done on chip instead:
//   warp 0      TMA producer: per window one tiled copy of the dense A window (As[KS][128],
//               unswizzled), one swizzled tiled copy per vector of its WS x 32
//               block of B (32-byte chunks swizzled within 128-byte rows: the one legal
//               layout of an MN-major TF32 operand), bulk copies of the packed indices and column_info lists.
//   warps 2-9   two sets of four gather warps that take the vectors in turn.  Thread = row
//               of the tile.  For one vector and window a thread reads its row's WS gathered
//               values from As (conflict-free: consecutive lanes, consecutive words) and
//               stores them as WS TMEM columns (tcgen05.st): the A operand of WS/8 MMAs.
//   warp 1      one thread issues tcgen05.mma kind::tf32, M128 N32 K8, A from TMEM, B from
//               shared memory, D = the vector's 32 accumulator columns in TMEM, and commits
//               to mbarriers that hand the A buffers and the stage back.
//   epilogue    the gather warps read the accumulators (tcgen05.ld) and store C.
// Every wait is bounded; a wait that gives up raises the device status word.
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"
#include "tcgen05.cuh"

namespace nmspmm {

template <int WS, int KS_, int MODE, int QT_>
struct Tf32Cfg {
    static constexpr int MS = 128, QT = QT_, NS = QT * 32;   // QT = 8: one CTA per SM; QT = 4: two
    static constexpr int KS = KS_;
    static constexpr int G = WS / 8;                       // MMAs (K = 8 each) per vector and window
    static_assert(WS % 8 == 0, "kind::tf32 contracts 8 rows per instruction");
    static constexpr int B_BYTES = QT * WS * 128;          // per vector WS rows of 128 bytes, swizzled; multiple of 1024
    static constexpr int A_BYTES = KS * MS * 4;
    static constexpr int D_BYTES = ((WS * (QT > 4 ? QT : 4) * 4 + 127) / 128) * 128;
    static constexpr int CI_BYTES = (MODE == kModeHigh) ? QT * 256 : 0;
    static constexpr int STAGE_BYTES = ((B_BYTES + A_BYTES + D_BYTES + CI_BYTES + 1023) / 1024) * 1024;
    static constexpr int CTAS_PER_SM = (QT == 8) ? 1 : 2;
    static constexpr int ST0 = ((CTAS_PER_SM == 1 ? 196 : 100) * 1024) / STAGE_BYTES;
    static constexpr int STAGES = ST0 > 4 ? 4 : (ST0 < 2 ? 2 : ST0);
    static constexpr int TMEM_COLS = 512 / CTAS_PER_SM;    // each resident CTA allocates its share
    static constexpr int NB0 = (TMEM_COLS - NS) / (2 * WS);
    static constexpr int NB = NB0 > 4 ? 4 : NB0;           // A buffers (WS TMEM columns each) per gather set
    static constexpr int GATHER_WARPS = 8;
    static constexpr int THREADS = (2 + GATHER_WARPS) * 32;
    static constexpr int TAB_BYTES = GATHER_WARPS * QT * WS * 4;   // per-warp table of gather offsets
    static constexpr int NBARS = 2 * STAGES + 4 * NB + 1;
    static constexpr int CTRL_BYTES = ((NBARS * 8 + 16 + 127) / 128) * 128;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + TAB_BYTES + CTRL_BYTES + 1024;   // + alignment slack
    static constexpr int ACOL0 = NS;                       // first A-buffer column
    static_assert(NB >= 1 && NS + 2 * NB * WS <= TMEM_COLS, "A buffers do not fit beside the accumulators");
    static constexpr bool HALF = false;
};

template <int WS, int KS_, int MODE, int QT_>
__global__ void __launch_bounds__((Tf32Cfg<WS, KS_, MODE, QT_>::THREADS), (Tf32Cfg<WS, KS_, MODE, QT_>::CTAS_PER_SM))
nm_gemm_tf32_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b)
{
    using Cfg = Tf32Cfg<WS, KS_, MODE, QT_>;
    constexpr int MS = Cfg::MS, NS = Cfg::NS, QT = Cfg::QT, KS = Cfg::KS, G = Cfg::G, STAGES = Cfg::STAGES, NB = Cfg::NB;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;          // swizzle atoms want 1024-byte alignment
    const uint32_t tabs = ring + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bars = tabs + Cfg::TAB_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + STAGES * 8;
    const uint32_t bar_aready = bar_empty + STAGES * 8, bar_afree = bar_aready + 2 * NB * 8;
    const uint32_t bar_acc = bar_afree + 2 * NB * 8;
    const uint32_t tmem_word = bar_acc + 8, abort_word = tmem_word + 4;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x;
    const int ty = tile / g.tiles_x, tx = tile - ty * g.tiles_x;
    const int bi = ty * MS, bj = tx * NS;
    const int n_win = g.sched.n_win;
    const int live_vecs = min(QT, (g.N - bj) / 32);        // vectors of the tile that exist
    const int qs_shift = g.qs_shift, layout_shift = qs_shift + 5;
    const int d_chunk = WS << qs_shift;
    const uint32_t d_bytes = static_cast<uint32_t>(d_chunk) * 4u;
    const int lb0 = bj >> layout_shift;
    const int nlb = ((bj + live_vecs * 32 - 1) >> layout_shift) - lb0 + 1;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, Cfg::GATHER_WARPS + 1);          // eight gather warps + the MMA commit
        }
        for (int b = 0; b < 2 * NB; ++b) {
            mbar_init(bar_aready + b * 8, 4);                             // the four warps of a set
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
            if (lane == 0) {
                mbar_arrive_expect_tx(full, Cfg::A_BYTES + live_vecs * (WS * 128) +
                                                nlb * (d_bytes + (MODE == kModeHigh ? 256u : 0u)));
                tma_load_2d(as, &map_a, bi, it * KS, full);
            }
            __syncwarp();
            if (lane < live_vecs) tma_load_2d(st + lane * (WS * 128), &map_b, bj + lane * 32, it * WS, full);
            if (lane < nlb) {
                const int* src = g.D + ((static_cast<size_t>(lb0 + lane) * g.W) << qs_shift) + static_cast<size_t>(it) * d_chunk;
                bulk_g2s(ds + lane * d_bytes, src, d_bytes, full);
                if (MODE == kModeHigh) {
                    const int* ci = g.cinfo + (static_cast<size_t>(lb0 + lane) * n_win + it) * 64;
                    bulk_g2s(ds + Cfg::D_BYTES + lane * 256, ci, 256, full);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = umma_idesc_tf32(128, 32);
        unsigned cnt0 = 0u, cnt1 = 0u;                     // units issued per gather set
        bool alive = true;
        for (int it = 0; it < n_win && alive; ++it) {
            const int s = it % STAGES;
            bool ok = mbar_wait_bounded(bar_full + s * 8, (it / STAGES) & 1, abort_word);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            const uint32_t st = ring + s * Cfg::STAGE_BYTES;
            int set = 0;
            for (int v = 0; v < live_vecs && alive; ++v) {
                // one chunk = the whole window of one vector: G MMAs on one A buffer
                const unsigned c = set ? cnt1 : cnt0;
                const int buf = set * NB + static_cast<int>(c % NB);
                ok = mbar_spin_bounded(bar_aready + buf * 8, (c / NB) & 1, abort_word);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { alive = false; break; }
                tc_fence_after_sync();
                if (lane == 0) {
#pragma unroll
                    for (int gi = 0; gi < G; ++gi)
                        umma_tf32_ts(tmem_addr(tmem, 0, v * 32), tmem_addr(tmem, 0, Cfg::ACOL0 + buf * WS + gi * 8),
                                     umma_desc_mn_tf32(st + v * (WS * 128) + gi * 1024), idesc, (it | gi) != 0);
                    tc_commit(bar_afree + buf * 8);        // the A buffer is free once these MMAs have read it
                }
                __syncwarp();
                if (set) ++cnt1; else ++cnt0;
                set ^= 1;
            }
            if (lane == 0) tc_commit(bar_empty + s * 8);   // the window's B blocks have been read
            __syncwarp();
        }
        if (!alive && lane == 0) atomicMax(g.status, kDevTimeoutMma);
        if (lane == 0) tc_commit(bar_acc);                 // every MMA has completed: accumulators are final
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ gather warps
        const int gw = warp - 2;                           // 0..7
        const int set = gw >> 2;                           // which set of four warps
        const int quad = warp & 3;                         // TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;                  // row of the tile this thread carries
        const uint32_t tab = tabs + gw * (QT * WS * 4);
        unsigned cnt = 0;                                  // units this set has produced
        bool alive = true;
        for (int it = 0; it < n_win && alive; ++it) {
            const int s = it % STAGES;
            bool ok = mbar_wait_bounded(bar_full + s * 8, (it / STAGES) & 1, abort_word);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            const uint32_t st = ring + s * Cfg::STAGE_BYTES;
            const uint32_t as = st + Cfg::B_BYTES, ds = as + Cfg::A_BYTES, cs = ds + Cfg::D_BYTES;
            // Resolve the window's indices to byte offsets of rows of As, once per warp.
            for (int e = lane; e < live_vecs * WS; e += 32) {
                const int v = e / WS, p = e - v * WS;
                const int q = (bj >> 5) + v;
                const int lb = (q >> qs_shift) - lb0;
                int k = lds_s32(ds + (lb * d_chunk + (p << qs_shift) + (q & ((1 << qs_shift) - 1))) * 4);
                if (MODE == kModeHigh) k = lds_s32(cs + (lb * 64 + k) * 4);
                sts_volatile_s32(tab + e * 4, k * (MS * 4));
            }
            __syncwarp();
            for (int v = set; v < live_vecs && alive; v += 2) {     // the two sets take the vectors in turn
                const int buf = set * NB + static_cast<int>(cnt % NB);
                if (cnt >= NB) {
                    ok = mbar_spin_bounded(bar_afree + buf * 8, ((cnt / NB) - 1) & 1, abort_word);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) { alive = false; break; }
                    tc_fence_after_sync();
                }
                const uint32_t base = as + row * 4;
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const int4 o0 = lds_i4(tab + (v * WS + gi * 8) * 4), o1 = lds_i4(tab + (v * WS + gi * 8 + 4) * 4);
                    uint32_t a[8];
                    a[0] = lds_u32(base + o0.x); a[1] = lds_u32(base + o0.y);
                    a[2] = lds_u32(base + o0.z); a[3] = lds_u32(base + o0.w);
                    a[4] = lds_u32(base + o1.x); a[5] = lds_u32(base + o1.y);
                    a[6] = lds_u32(base + o1.z); a[7] = lds_u32(base + o1.w);
                    tmem_st_x8(tmem_addr(tmem, quad * 32, Cfg::ACOL0 + buf * WS + gi * 8), a);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_aready + buf * 8);
                ++cnt;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);     // this warp has finished reading As of the stage
        }
        // ------------------------------------------------------------------ epilogue
        bool ok = alive && mbar_wait_bounded(bar_acc, 0, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
            const int r = bi + row;
            const int half = gw >> 2;                      // lower or upper half of the tile's columns
#pragma unroll 1
            for (int c = 0; c < QT / 2; ++c) {
                const int col = half * (NS / 2) + c * 32;
                if (col >= live_vecs * 32) break;
                uint32_t v[32];
                tmem_ld_x32(tmem_addr(tmem, quad * 32, col), v);
                tmem_wait_ld();
                if (r < g.M) {
                    float4* dst = reinterpret_cast<float4*>(g.C + static_cast<size_t>(r) * g.N + bj + col);
#pragma unroll
                    for (int x = 0; x < 8; ++x)
                        dst[x] = make_float4(__uint_as_float(v[4 * x]), __uint_as_float(v[4 * x + 1]),
                                             __uint_as_float(v[4 * x + 2]), __uint_as_float(v[4 * x + 3]));
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
static cudaError_t launch_tf32(const GemmArgs& a, int tiles, cudaStream_t st)
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
    kernel<<<tiles, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(a, map_a, map_b);
    return cudaGetLastError();
}

#define NMSPMM_TF32_VARIANT(NKEEP, WS, KS, MODE, QT)                                                        \
    { NKEEP, WS, KS, MODE, QT * 32, Tf32Cfg<WS, KS, MODE, QT>::SMEM_BYTES, Tf32Cfg<WS, KS, MODE, QT>::STAGES, \
      &launch_tf32<WS, KS, MODE, QT> }

extern const Tf32Variant kTf32Variants[] = {
    NMSPMM_TF32_VARIANT(32, 32, 32, kModeLow, 8),  NMSPMM_TF32_VARIANT(32, 32, 32, kModeLow, 4),
    NMSPMM_TF32_VARIANT(16, 16, 32, kModeLow, 8),  NMSPMM_TF32_VARIANT(16, 16, 32, kModeLow, 4),
    NMSPMM_TF32_VARIANT(8, 8, 32, kModeLow, 8),    NMSPMM_TF32_VARIANT(8, 8, 32, kModeLow, 4),
    NMSPMM_TF32_VARIANT(8, 16, 64, kModeHigh, 8),  NMSPMM_TF32_VARIANT(8, 16, 64, kModeHigh, 4),
    NMSPMM_TF32_VARIANT(4, 8, 64, kModeHigh, 8),   NMSPMM_TF32_VARIANT(4, 8, 64, kModeHigh, 4),
};
extern const int kTf32VariantCount = sizeof(kTf32Variants) / sizeof(kTf32Variants[0]);

}  // namespace nmspmm
