// TF32 tensor-core path of the vector-wise N:M sparse GEMM (tcgen05, accumulators in TMEM).
//
// One CTA computes a 128 x NS tile of C (QT = NS / 32 vectors of 32 columns) over its k steps.
// A step is one 32-k window (one 64-k merged window for 4:32) with WS kept rows of B.  The
// contraction is per vector, C[128 x 32] += A_gathered[128 x WS] . B[WS x 32], and A_gathered
// (the WS columns of the step's A window that the vector's index list names) differs for
// every vector.  The gather itself is done by the tensor core:
//
//     G[128 x QT*WS] = A_window[128 x KW] . P[KW x QT*WS]
//
// where column (v, j) of P is one-hot at the k that vector v's j-th index names.  Products
// with 1.0 and sums with 0.0 are exact, so G holds exactly the (TF32-truncated) gathered
// values -- in Tensor Memory, lane = tile row, column = (v, j): the layout of a TMEM A
// operand.  The second instruction group then multiplies, per vector, G's WS columns by the
// vector's WS x 32 block of B.  Nothing of A goes through registers; the only generic-proxy
// shared-memory traffic of the main loop is two 4-byte stores per index (clear the old
// one-hot entry, set the new one).  Tensor work is twice the useful work for every ratio.
// A non-finite value anywhere in a row of the A window reaches every gathered column of that
// row (0 x inf), not only the vectors that select it: this path wants finite A.
//
//   warp 0      TMA producer: per step one tiled copy of the A window and one of the B rows,
//               both as blocks of 32 floats along m / n with 32-byte chunks swizzled within
//               128-byte rows (the one legal layout of an MN-major TF32 operand).
//   warp 1      one elected thread issues the gathers (tcgen05.mma kind::tf32, A and P from
//               shared memory, M128 N=QT*WS, KW/8 instructions per step) into a ring of
//               result buffers in TMEM, each followed by a tcgen05.commit to the buffer's
//               mbarrier.
//   warps 2-3   one elected thread each issues the products of half the tile's vectors
//               (A = G from TMEM, B from shared memory, M128 N32 K8 each) once the gather's
//               mbarrier has completed, and commits to the mbarrier that frees the stage and
//               the result buffer.  One thread issues a tcgen05.mma every 26 cycles at best
//               (measured), and a step has 12 to 20 of them: three issuing threads keep the
//               tensor pipe, not the issue slot, the bound.
//   warps 4-7   one thread per (vector, kept row): fetches its index two to four steps ahead
//               with cp.async (through column_info on the 64-k format), keeps P's one-hot
//               entry current, and after the last step reads the accumulators (tcgen05.ld),
//               transposes them through shared memory and stores C in 128-byte row pieces.
// n_keep = 32 (nothing pruned) has the identity as its index list and multiplies A_window by
// the B rows directly.  12:32 gathers 16 columns per vector of which 4 are zero (P has no
// entry for them), and loads 16 rows of B per vector of which the last 4 meet those zeros.
// Every wait is bounded; a wait that gives up raises the device status word.
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"
#include "tcgen05.cuh"
#include "tf32_epilogue.cuh"

namespace nmspmm {

// Diagnostic target, not part of the shipped library: built with
//     NMSPMM_NVCC_EXTRA=-DNMSPMM_TF32_PROFILE NMSPMM_BUILD_DIR=<dir> NMSPMM_BUILD_LIB=<file.so> python nm-spmm_b200/build.py
// the kernel adds up, per role, the cycles (clock64) spent waiting and issuing, and
// nmspmm_debug_tf32_profile (exported by that build only) reads and clears the sixteen sums:
//   0 producer waits for a free stage, 1 producer total, 2 / 3 / 4 / 5 gather issuer: wait for the
//   stage, wait for a result buffer, issue, total, 6 / 7 / 15 product issuer: wait for the gather,
//   issue, total, 8 CTAs, 9 steps, 13 / 14 epilogue: wait for the accumulators, run.
// Without the macro every TF_* below expands to nothing.
#ifdef NMSPMM_TF32_PROFILE
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

template <int NKEEP, int KW_, int MODE, int QT_, int VL_ = 32>
struct Tf32Cfg {
    static constexpr int MS = 128, QT = QT_, NS = QT * 32;   // QT = 8: one CTA per SM; QT = 4: two
    static constexpr int KW = KW_;                           // k per step
    static constexpr int WS = NKEEP * (KW / 32);             // rows of B per step
    static constexpr int WSP = (WS + 7) / 8 * 8;             // gathered columns per vector (K of the products)
    static constexpr bool DIRECT = (NKEEP == 32);            // identity index list: no gather
    static constexpr int G = WSP / 8;                        // product instructions per vector and step
    static constexpr int NKS = KW / 8;                       // gather instructions per step
    static constexpr int VL = VL_;                           // columns that share an index list: 32, or 64 (two adjacent equal lists)
    static constexpr int QV = NS / VL;                       // vectors per tile
    static constexpr int N1 = QV * WSP;                      // gathered columns per step
    static_assert(VL == 32 || (VL == 64 && NKEEP != 32), "vectors of 32 or 64 columns");
    static_assert(DIRECT || N1 <= 128, "one builder thread per gathered column");
    static_assert(MODE == kModeHigh || KW == 32, "only the 64-k format has merged windows");
    static constexpr int A_BYTES = KW * 512;                 // [4 blocks of 32 rows of the tile][KW][32]
    static constexpr int B_BYTES = QT * WSP * 128;           // [QT][WSP][32]
    static constexpr int P_BYTES = DIRECT ? 0 : N1 * KW * 4; // [N1 / 32][KW][32]
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + P_BYTES;
    static_assert(A_BYTES % 1024 == 0 && B_BYTES % 1024 == 0 && P_BYTES % 1024 == 0, "swizzle atoms stay aligned");
    static constexpr int CTAS_PER_SM = (QT == 8) ? 1 : 2;
    static constexpr int TMEM_COLS = 512 / CTAS_PER_SM;      // each resident CTA allocates its share
    static constexpr int PD = 2;                             // index prefetch distance, in steps, per look-up
    static constexpr int RING = 4 * PD;                      // slots of the per-thread index rings
    static constexpr int BUILDERS = 128;
    static constexpr int PRODUCT_WARPS = 2;
    static constexpr int THREADS = (2 + PRODUCT_WARPS) * 32 + BUILDERS;
    static constexpr int AUX_BYTES = (2 * RING + 8) * BUILDERS * 4;    // index rings + previous one-hot per stage (<= 8 stages)
    static constexpr int CTRL_BYTES = 256;
    static constexpr int SMEM_LIMIT = (CTAS_PER_SM == 1 ? 227 : 113) * 1024;
    static constexpr int ST0 = (SMEM_LIMIT - 1024 - AUX_BYTES - CTRL_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = ST0 > 6 ? 6 : ST0;
    static_assert(STAGES >= 2, "at least two stages");
    // Ring of gather results beside the accumulators.  A gather's result is complete (and its
    // commit arrives) some hundreds of cycles after issue, and the products that free the
    // buffer again take as long: the loop gather -> products -> gather is latency-bound
    // unless several steps are in flight, so the ring is as deep as Tensor Memory allows.
    static constexpr int NBUF0 = DIRECT ? 1 : (TMEM_COLS - NS) / N1;
    static constexpr int NBUF = NBUF0 > 4 ? 4 : NBUF0;
    static_assert(NBUF >= 1, "no room for a gather result beside the accumulators");
    static constexpr int EPI_BYTES = 4 * kTf32PatchBytes;    // four warps' transposition patches
    static_assert(EPI_BYTES <= STAGES * STAGE_BYTES, "the epilogue reuses the stage ring");
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + CTRL_BYTES + 1024;   // + alignment slack
    static constexpr int ACOL0 = NS;                         // first gather-result column
};

// Byte offset of P[k][n] (n = gathered column) inside a stage's P region.
template <int KW>
__device__ __forceinline__ uint32_t p_offset(int n, int k)
{
    const int nb = n >> 5, c = n & 31;
    return static_cast<uint32_t>(nb * (KW * 128) + k * 128 + ((((c >> 3) ^ (k & 3)) << 5) | ((c & 7) << 2)));
}

template <int NKEEP, int KW_, int MODE, int QT_, int VL_>
__global__ void __launch_bounds__((Tf32Cfg<NKEEP, KW_, MODE, QT_, VL_>::THREADS), (Tf32Cfg<NKEEP, KW_, MODE, QT_, VL_>::CTAS_PER_SM))
nm_gemm_tf32_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmOutputs outs, const int a_blocked)
{
    using Cfg = Tf32Cfg<NKEEP, KW_, MODE, QT_, VL_>;
    constexpr int MS = Cfg::MS, NS = Cfg::NS, QT = Cfg::QT, KW = Cfg::KW, WS = Cfg::WS, WSP = Cfg::WSP;
    constexpr int VL = Cfg::VL, QV = Cfg::QV, BPV = VL / 32;              // 32-column blocks per vector
    constexpr int STAGES = Cfg::STAGES, NBUF = Cfg::NBUF, RING = Cfg::RING, PD = Cfg::PD;
    constexpr bool DIRECT = Cfg::DIRECT;
    constexpr int FIRST_BUILDER = 2 + Cfg::PRODUCT_WARPS;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;          // swizzle atoms want 1024-byte alignment
    const uint32_t idx_ring = ring + STAGES * Cfg::STAGE_BYTES;           // [RING][128] raw index (rank on the 64-k format)
    const uint32_t k_ring = idx_ring + RING * 512;                        // [RING][128] k after the column_info look-up
    const uint32_t prev_k = k_ring + RING * 512;                          // [STAGES][128] one-hot entry now set in the stage
    const uint32_t bars = ring + STAGES * Cfg::STAGE_BYTES + Cfg::AUX_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + STAGES * 8;
    const uint32_t bar_gdone = bar_empty + STAGES * 8, bar_gfree = bar_gdone + 4 * 8, bar_acc = bar_gfree + 4 * 8;
    const uint32_t tmem_word = bar_acc + 8, abort_word = tmem_word + 4;
    static_assert((2 * 6 + 2 * 4 + 1) * 8 + 8 <= Cfg::CTRL_BYTES, "control block");

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
    int ty, tx;
    tile_coords(tile, g.tiles_x, (g.M + MS - 1) / MS, ty, tx);
    const int bi = ty * MS, bj = tx * NS;
    int win0, n_win;                                       // this CTA's steps: win0 .. win0 + n_win - 1
    slice_range(g.sched.n_win, n_slices, sliced ? slot % n_slices : 0, win0, n_win);
    const int live_vecs = min(QT, (g.N - bj) / 32);        // vectors of the tile that exist

    if (tid == 0) {
        prefetch_tensor_map(&map_a);
        prefetch_tensor_map(&map_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, DIRECT ? 1 : 1 + Cfg::BUILDERS / 32);   // the TMA bytes + the builder warps
            mbar_init(bar_empty + s * 8, DIRECT ? 1 : Cfg::PRODUCT_WARPS);      // the commits behind the step's products
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(bar_gdone + b * 8, 1);                                    // the commit behind a gather
            mbar_init(bar_gfree + b * 8, Cfg::PRODUCT_WARPS);                   // the commits behind the products that read it
        }
        mbar_init(bar_acc, DIRECT ? 1 : Cfg::PRODUCT_WARPS);
        sts_volatile_s32(abort_word, 0);
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_word, Cfg::TMEM_COLS);
    if (!DIRECT) {
        // P starts as all zeros; 12:32 also wants the never-set columns of every vector zero
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < STAGES; ++s)
            for (int o = tid * 16; o < Cfg::P_BYTES; o += Cfg::THREADS * 16)
                sts_f4(ring + s * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::B_BYTES + o, z);
        fence_proxy_async();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = static_cast<uint32_t>(lds_volatile_s32(tmem_word));
    grid_dependency_wait();                                // everything above overlapped the tail of the kernel ahead

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        TF_DECL(p_empty = 0);
        TF_T(p_start);
        for (int it = 0; it < n_win; ++it) {
            const int s = it % STAGES;
            if (it >= STAGES) {
                TF_T(t0);
                const bool ok = mbar_wait_bounded(bar_empty + s * 8, ((it / STAGES) - 1) & 1, abort_word);
                TF_ADD(p_empty, t0);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicMax(g.status, kDevTimeoutEmpty);
                    break;
                }
            }
            const uint32_t st = ring + s * Cfg::STAGE_BYTES, full = bar_full + s * 8;
            if (elect_one()) {
                mbar_arrive_expect_tx(full, Cfg::A_BYTES + Cfg::B_BYTES);
                if (a_blocked) {
                    tma_load_3d(st, &map_a, 0, (win0 + it) * KW, bi >> 5, full);
                } else {                                   // rows not a multiple of 32: four boxes of 32 rows, the ragged one zero-filled
                    for (int mb = 0; mb < 4; ++mb) tma_load_2d(st + mb * (KW * 128), &map_a, bi + mb * 32, (win0 + it) * KW, full);
                }
                tma_load_3d(st + Cfg::A_BYTES, &map_b, 0, (win0 + it) * WS, bj >> 5, full);
            }
            __syncwarp();
        }
#ifdef NMSPMM_TF32_PROFILE
        if (lane == 0) { TF_OUT(0, p_empty); TF_OUT(1, clock64() - p_start); }
#endif
    } else if (warp == 1) {
        // ------------------------------------------------------------------ gather issuer
        constexpr uint32_t idesc_gather = umma_idesc_tf32(128, DIRECT ? 32 : Cfg::N1, true);
        const uint32_t idesc_direct = umma_idesc_tf32(128, live_vecs * 32, true);
        bool alive = true;
        TF_DECL(m_full = 0, m_free = 0, m_issue = 0);
        TF_T(m_start);
        for (int t = 0; t < n_win; ++t) {
            const int s = t % STAGES;
            TF_T(t0);
            bool ok = mbar_wait_bounded(bar_full + s * 8, (t / STAGES) & 1, abort_word);
            TF_ADD(m_full, t0);
            TF_T(t1);
            if (!DIRECT && t >= NBUF)                      // the result buffer is free once the products of step t - NBUF are done
                ok = ok && mbar_wait_bounded(bar_gfree + (t % NBUF) * 8, ((t / NBUF) - 1) & 1, abort_word);
            TF_ADD(m_free, t1);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            TF_T(t2);
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t st = ring + s * Cfg::STAGE_BYTES;
                if (DIRECT) {
#pragma unroll
                    for (int ks = 0; ks < Cfg::NKS; ++ks)
                        umma_tf32_ss(tmem_addr(tmem, 0, 0), umma_desc_mn_tf32(st + ks * 1024, KW * 128, 512),
                                     umma_desc_mn_tf32(st + Cfg::A_BYTES + ks * 1024, WSP * 128, 512), idesc_direct,
                                     (t | ks) != 0);
                    tc_commit(bar_empty + s * 8);
                } else {
                    const uint32_t gbuf = tmem_addr(tmem, 0, Cfg::ACOL0 + (t % NBUF) * Cfg::N1);
#pragma unroll
                    for (int ks = 0; ks < Cfg::NKS; ++ks)
                        umma_tf32_ss(gbuf, umma_desc_mn_tf32(st + ks * 1024, KW * 128, 512),
                                     umma_desc_mn_tf32(st + Cfg::A_BYTES + Cfg::B_BYTES + ks * 1024, KW * 128, 512),
                                     idesc_gather, ks != 0);
                    tc_commit(bar_gdone + (t % NBUF) * 8);
                }
            }
            __syncwarp();
            TF_ADD(m_issue, t2);
        }
#ifdef NMSPMM_TF32_PROFILE
        if (lane == 0) {
            TF_OUT(2, m_full); TF_OUT(3, m_free); TF_OUT(4, m_issue); TF_OUT(5, clock64() - m_start); TF_OUT(8, 1); TF_OUT(9, n_win);
        }
#endif
        if (!alive && lane == 0) atomicMax(g.status, kDevTimeoutMma);
        if (DIRECT) {
            if (elect_one()) tc_commit(bar_acc);           // every MMA has completed: accumulators are final
            __syncwarp();
        }
    } else if (warp < FIRST_BUILDER) {
        // ------------------------------------------------------------------ product issuers
        if (!DIRECT) {
            constexpr uint32_t idesc_product = umma_idesc_tf32(128, VL, false);
            constexpr int VPI = QV / Cfg::PRODUCT_WARPS;   // vectors per issuer
            const int v_begin = (warp - 2) * VPI, v_end = min(v_begin + VPI, live_vecs / BPV);
            bool alive = true;
            TF_DECL(c_gdone = 0, c_issue = 0);
            TF_T(c_start);
            for (int u = 0; u < n_win; ++u) {
                const int s = u % STAGES, b = u % NBUF;
                TF_T(t0);
                // the step's B rows have landed (their barrier completed before the gather was issued)
                bool ok = mbar_wait_bounded(bar_full + s * 8, (u / STAGES) & 1, abort_word);
                ok = ok && mbar_spin_bounded(bar_gdone + b * 8, (u / NBUF) & 1, abort_word);
                TF_ADD(c_gdone, t0);
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                TF_T(t1);
                tc_fence_after_sync();
                if (elect_one()) {
                    if (v_begin < v_end) {
                        const uint32_t bs = ring + s * Cfg::STAGE_BYTES + Cfg::A_BYTES;
                        const uint32_t gbuf = tmem_addr(tmem, 0, Cfg::ACOL0 + b * Cfg::N1);
                        for (int v = v_begin; v < v_end; ++v) {
#pragma unroll
                            for (int gi = 0; gi < Cfg::G; ++gi)
                                umma_tf32_ts(tmem_addr(tmem, 0, v * VL), gbuf + v * WSP + gi * 8,
                                             umma_desc_mn_tf32(bs + v * (BPV * WSP * 128) + gi * 1024, WSP * 128, 512),
                                             idesc_product, (u | gi) != 0);
                        }
                        tc_commit(bar_empty + s * 8);      // this half of the step's products has read the stage
                        tc_commit(bar_gfree + b * 8);      // and the gather result
                    } else {
                        mbar_arrive(bar_empty + s * 8);    // no vector of this half exists; the gather itself has completed
                        mbar_arrive(bar_gfree + b * 8);
                    }
                }
                __syncwarp();
                TF_ADD(c_issue, t1);
            }
#ifdef NMSPMM_TF32_PROFILE
            if (lane == 0 && warp == 2) { TF_OUT(6, c_gdone); TF_OUT(7, c_issue); TF_OUT(15, clock64() - c_start); }
#endif
            if (!alive && lane == 0) atomicMax(g.status, kDevTimeoutMma);
            if (elect_one()) {
                if (v_begin < v_end) tc_commit(bar_acc); else mbar_arrive(bar_acc);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ one-hot builders
        const int e = tid - FIRST_BUILDER * 32;            // gathered column this thread keeps
        const int quad = warp & 3;                         // TMEM lane quadrant this warp may touch
        bool alive = true;
        if (!DIRECT) {
            const int v = e / WSP, j = e % WSP;
            const bool has = e < Cfg::N1 && j < WS && v * BPV < live_vecs;
            const int q = (bj >> 5) + v * BPV, qs_shift = g.qs_shift;       // the (first) 32-column index list of vector v
            const int* dptr = g.D + ((static_cast<size_t>(q >> qs_shift) * g.W) << qs_shift) + (q & ((1 << qs_shift) - 1)) +
                              (static_cast<size_t>(j) << qs_shift);
            const int n_merged = (KW == 64) ? g.sched.n_win : (g.sched.n_win >> 1);
            const int* ciptr = (MODE == kModeHigh) ? g.cinfo + static_cast<size_t>(q >> qs_shift) * n_merged * 64 : nullptr;
            const uint32_t my_idx = idx_ring + e * 4, my_k = k_ring + e * 4, my_prev = prev_k + e * 4;
            for (int s = 0; s < STAGES; ++s) sts_s32(my_prev + s * 512, -1);
            TF_DECL(b_cp = 0, b_empty = 0);
            TF_T(b_start);
            for (int i = -2 * PD; i < n_win; ++i) {
                TF_T(t0);
                cp_async_wait<PD - 1>();                   // the copies issued PD iterations ago and earlier have landed
                TF_ADD(b_cp, t0);
                int k = 0;
                if (has && i >= 0) {
                    k = lds_s32((MODE == kModeHigh ? my_k : my_idx) + (i & (RING - 1)) * 512);
                    if (MODE == kModeHigh && KW == 32) k -= ((win0 + i) & 1) * 32;
                }
                if (has) {
                    const int i2 = i + 2 * PD, i1 = i + PD;
                    if (i2 < n_win)
                        cp_async_4(my_idx + (i2 & (RING - 1)) * 512, dptr + ((static_cast<size_t>(win0 + i2) * WS) << qs_shift));
                    if (MODE == kModeHigh && i1 >= 0 && i1 < n_win) {
                        const int rank = lds_s32(my_idx + (i1 & (RING - 1)) * 512);
                        const int m = (KW == 64) ? (win0 + i1) : ((win0 + i1) >> 1);
                        cp_async_4(my_k + (i1 & (RING - 1)) * 512, ciptr + static_cast<size_t>(m) * 64 + rank);
                    }
                }
                cp_async_commit();
                if (i < 0) continue;
                const int s = i % STAGES;
                if (i >= STAGES) {
                    TF_T(t1);
                    const bool ok = mbar_wait_bounded(bar_empty + s * 8, ((i / STAGES) - 1) & 1, abort_word);
                    TF_ADD(b_empty, t1);
                    if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                }
                if (has) {
                    const uint32_t ps = ring + s * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::B_BYTES;
                    const int old = lds_s32(my_prev + s * 512);
                    if (old >= 0) sts_f32(ps + p_offset<KW>(e, old), 0.f);
                    sts_f32(ps + p_offset<KW>(e, k), 1.f);
                    sts_s32(my_prev + s * 512, k);
                }
                fence_proxy_async();                       // the tensor core reads P through the asynchronous proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + s * 8);
            }
            cp_async_wait<0>();
#ifdef NMSPMM_TF32_PROFILE
            (void)b_cp; (void)b_empty; (void)b_start;
#endif
        }
        // ------------------------------------------------------------------ epilogue
        TF_T(e_start);
        bool ok = alive && mbar_wait_bounded(bar_acc, 0, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        grid_launch_dependents();                          // only stores are left
        TF_T(e_go);
        if (ok) {
            tc_fence_after_sync();
            // every MMA has completed, so every TMA copy has landed and been read: the
            // stage ring is free and serves as the transposition patches
            tf32_store_vectors<NS>(tmem, quad, lane, 0, live_vecs, ring + (warp - FIRST_BUILDER) * kTf32PatchBytes, g, outs, bi, bj,
                                   sliced, slot);
        } else if (lane == 0) {
            atomicMax(g.status, kDevTimeoutMma);
        }
#ifdef NMSPMM_TF32_PROFILE
        if (e == 0) { TF_OUT(13, e_go - e_start); TF_OUT(14, clock64() - e_go); }
#endif
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::TMEM_COLS);
    }
}

template <int NKEEP, int KW, int MODE, int QT, int VL>
static cudaError_t launch_tf32(const GemmArgs& a, const GemmOutputs& outs, int tiles, cudaStream_t st)
{
    using Cfg = Tf32Cfg<NKEEP, KW, MODE, QT, VL>;
    auto kernel = nm_gemm_tf32_kernel<NKEEP, KW, MODE, QT, VL>;
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
    const int K = a.sched.n_win * KW;
    const int lda = outs.lda ? outs.lda : a.M;             // a row-major caller's transposed copy is padded to 4 columns
    const int a_blocked = (lda % 32 == 0) ? 1 : 0;
    e = a_blocked ? encode_tensor_map_blocks32(&map_a, a.A, lda, K, KW, 4)
                  : encode_tensor_map_2d(&map_a, a.A, lda, K, 32, KW, 1);
    if (e != cudaSuccess) return e;
    e = encode_tensor_map_blocks32(&map_b, a.B, a.N, a.W, Cfg::WSP - (g_test_short_fill ? 1 : 0), QT);   // (test hook, see kernels.h)
    if (e != cudaSuccess) return e;
    return launch_overlapped(kernel, tiles, Cfg::THREADS, Cfg::SMEM_BYTES, st, a, map_a, map_b, outs, a_blocked);
}

#define NMSPMM_TF32_VARIANT(NKEEP, KW, MODE, QT, VL)                                                                   \
    { NKEEP, Tf32Cfg<NKEEP, KW, MODE, QT, VL>::WS, KW, MODE, QT * 32, VL, Tf32Cfg<NKEEP, KW, MODE, QT, VL>::SMEM_BYTES,    \
      Tf32Cfg<NKEEP, KW, MODE, QT, VL>::STAGES, Tf32Cfg<NKEEP, KW, MODE, QT, VL>::THREADS, &launch_tf32<NKEEP, KW, MODE, QT, VL> }

extern const SlicedVariant kTf32GatherVariants[] = {
    NMSPMM_TF32_VARIANT(32, 32, kModeLow, 8, 32),  NMSPMM_TF32_VARIANT(32, 32, kModeLow, 4, 32),
    NMSPMM_TF32_VARIANT(16, 32, kModeLow, 8, 32),  NMSPMM_TF32_VARIANT(16, 32, kModeLow, 4, 32),
    NMSPMM_TF32_VARIANT(12, 32, kModeLow, 8, 32),  NMSPMM_TF32_VARIANT(12, 32, kModeLow, 4, 32),
    NMSPMM_TF32_VARIANT(8, 32, kModeLow, 8, 32),   NMSPMM_TF32_VARIANT(8, 32, kModeLow, 4, 32),
    NMSPMM_TF32_VARIANT(8, 32, kModeHigh, 8, 32),  NMSPMM_TF32_VARIANT(8, 32, kModeHigh, 4, 32),
    NMSPMM_TF32_VARIANT(4, 64, kModeHigh, 8, 32),  NMSPMM_TF32_VARIANT(4, 64, kModeHigh, 4, 32),
    // vectors of 64 columns (two adjacent equal index lists): one gather and one N = 64 product per pair
    NMSPMM_TF32_VARIANT(16, 32, kModeLow, 8, 64),  NMSPMM_TF32_VARIANT(12, 32, kModeLow, 8, 64),
    NMSPMM_TF32_VARIANT(8, 32, kModeLow, 8, 64),   NMSPMM_TF32_VARIANT(8, 32, kModeHigh, 8, 64),
    NMSPMM_TF32_VARIANT(4, 64, kModeHigh, 8, 64),
};
extern const int kTf32GatherVariantCount = sizeof(kTf32GatherVariants) / sizeof(kTf32GatherVariants[0]);

#ifdef NMSPMM_TF32_PROFILE
// Diagnostic build only: reads and clears the phase counters.
extern "C" int nmspmm_debug_tf32_profile(unsigned long long* out16)
{
    if (cudaMemcpyFromSymbol(out16, g_tf32_profile, sizeof(unsigned long long) * 16) != cudaSuccess) return 1;
    unsigned long long zero[16] = {};
    return cudaMemcpyToSymbol(g_tf32_profile, zero, sizeof(zero)) == cudaSuccess ? 0 : 1;
}
#endif

}  // namespace nmspmm
