// TF32 path for few rows of A (M <= 64: the decode and small-batch shapes of a linear layer).
//
// These shapes are bound by streaming B once.  The tcgen05 tiles of gemm_tf32.cu work on 128
// rows whatever M is and a k step costs them about 600 cycles of instruction issue: three times
// the HBM time of B at 16 x 11008 x 4096.  Here: tile MS x 128 with MS = 16, 32 or 64, four
// warps = the tile's four vectors, K cut into slices so that every SM holds a few CTAs with
// their own TMA rings, and warp-level mma.sync.m16n8k8 (TF32 operands, FP32 accumulators in
// registers).  A fragment of A is four shared loads at the k rows the vector's index list names
// -- the gather is the address -- and serves the vector's four n8 blocks: a k8 group costs a
// warp 4 MS/16 + 8 shared loads and 4 MS/16 instructions.  The operands are FP32 bit patterns
// of which the tensor core uses the upper 19 bits, as on the tcgen05 path.
// (The same structure with an exact inner loop -- lane = column, MS accumulators, packed FMA,
// A by broadcast 16-byte loads -- was built and is slower than the register-tiled kernels of
// gemm_ffma.cuh at every shape tried, 24.3 against 20.8 us at 16 x 11008 x 4096 and 66 against
// 42 us at 64 rows: MS / 4 loads per MS / 2 instructions keep it on the load/store pipe.)
//
//   * The A window ([KS][16] as it lies in memory for 16 rows, else blocks [KS][32 rows of A])
//     and the B rows of the window as four blocks [WS][32], the blocks with 32-byte chunks
//     swizzled within 128-byte rows (fragment loads of lanes that read different k then fall
//     into different banks unless their k agree modulo 4), arrive by TMA in a ring of STAGES
//     slots; one thread refills a slot after the CTA's barrier behind its window.
//   * The k of every kept row of the CTA's windows (through column_info on the 64-k formats)
//     is resolved once, before the loop, into shared memory: a window's arithmetic is far
//     shorter than a trip to L2.
//   * K slices of a tile leave their accumulators in scratch slots of MS x 128 floats and
//     nm_reduce_slices_kernel adds them in k order; a tile computed by one CTA is stored
//     directly (to every output buffer when the caller gathers).
// Every wait is bounded; a wait that gives up raises the device status word.
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"

namespace nmspmm {

template <int MS_, int WS_, int KS_, int MODE_>
struct FewRowsCfg {
    static constexpr int MS = MS_, NS = 128, WS = WS_, KS = KS_, MODE = MODE_;
    static constexpr int THREADS = 128, MB = MS / 16, GROUPS = WS / 8;
    static constexpr bool A_PLAIN = (MS == 16);              // 16 rows: [KS][16] as it lies in memory; else swizzled blocks of 32 rows
    static constexpr int ABLK = (MS + 31) / 32;
    static constexpr int A_BYTES = A_PLAIN ? KS * 64 : ABLK * KS * 128;
    static constexpr int B_BYTES = 4 * WS * 128;             // [4 vectors][WS][32]
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (MS == 16) ? 4 : ((MS == 32) ? 3 : 2);   // four CTAs per SM in every case
    static constexpr int MAX_WINDOWS = kFewRowsMaxWindows;   // windows of one CTA (the planner cuts K accordingly)
    static constexpr int K_BYTES = MAX_WINDOWS * 4 * WS * 4; // resolved k of every kept row: [window][vector][WS]
    static constexpr int CTRL_BYTES = 128;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + K_BYTES + CTRL_BYTES + 1024;   // + alignment slack
    static constexpr int MIN_BLOCKS = (227 * 1024) / (SMEM_BYTES + 1024) > 4 ? 4 : (227 * 1024) / (SMEM_BYTES + 1024);
    static_assert(MS % 16 == 0 && WS % 8 == 0 && A_BYTES % 512 == 0 && B_BYTES % 512 == 0, "fragment shapes, swizzle period");
    static_assert((MODE == kModeHigh) == (KS == 64), "the 64-k formats have merged windows");
};

__device__ __forceinline__ void mma_tf32_16x8x8(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MS_, int WS_, int KS_, int MODE_>
__global__ void __launch_bounds__(128, (FewRowsCfg<MS_, WS_, KS_, MODE_>::MIN_BLOCKS))
nm_gemm_tf32_few_rows_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const GemmOutputs outs, const int a_blocked)
{
    using Cfg = FewRowsCfg<MS_, WS_, KS_, MODE_>;
    constexpr int MS = Cfg::MS, NS = Cfg::NS, WS = Cfg::WS, KS = Cfg::KS, MB = Cfg::MB, STAGES = Cfg::STAGES;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t k_list = ring + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_full = k_list + Cfg::K_BYTES, abort_word = bar_full + STAGES * 8;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
    const int S = g.sched.split_k;                         // K slices per tile (>= 1); CTA = (tile, slice)
    const int tile = static_cast<int>(blockIdx.x) / S, z = static_cast<int>(blockIdx.x) - tile * S;
    const int bj = tile * NS;                              // one row of tiles: M <= MS
    int win0, n_win;
    slice_range(g.sched.n_win, S, z, win0, n_win);
    const int live_vecs = min(4, (g.N - bj) / 32);

    if (tid == 0) {
        prefetch_tensor_map(&map_a);
        prefetch_tensor_map(&map_b);
        for (int s = 0; s < STAGES; ++s) mbar_init(bar_full + s * 8, 1);
        sts_volatile_s32(abort_word, 0);
        mbar_init_fence();
    }
    __syncthreads();
    grid_dependency_wait();                                // everything above overlapped the tail of the kernel ahead

    auto fill = [&](int it) {                              // one thread: the copies of window win0 + it into slot it % STAGES
        const int s = it % STAGES;
        const uint32_t dst = ring + s * Cfg::STAGE_BYTES, full = bar_full + s * 8;
        mbar_arrive_expect_tx(full, Cfg::STAGE_BYTES);
        if (Cfg::A_PLAIN) {
            tma_load_2d(dst, &map_a, 0, (win0 + it) * KS, full);
        } else if (a_blocked) {
            tma_load_3d(dst, &map_a, 0, (win0 + it) * KS, 0, full);
        } else {                                           // rows of A not a multiple of 32: one box per block, the ragged one zero-filled
            for (int blk = 0; blk < Cfg::ABLK; ++blk) tma_load_2d(dst + blk * (KS * 128), &map_a, blk * 32, (win0 + it) * KS, full);
        }
        tma_load_3d(dst + Cfg::A_BYTES, &map_b, 0, (win0 + it) * WS, bj >> 5, full);
    };
    if (tid == 0)
        for (int it = 0; it < STAGES && it < n_win; ++it) fill(it);

    // k of every kept row of this CTA's windows, entry (window, vector, j): first all raw indices,
    // then (64-k formats) all look-ups of the merged windows' column lists -- two trips to L2 for
    // the CTA, not two per entry
    {
        const int qs_shift = g.qs_shift, q0 = bj >> 5, n_e = n_win * 4 * WS;
#pragma unroll 4
        for (int e = tid; e < n_e; e += Cfg::THREADS) {
            const int j = e % WS, v = (e / WS) & 3, w = e / (4 * WS);
            int k = 0;
            if (v < live_vecs) {
                const int q = q0 + v;
                const int* dptr = g.D + ((static_cast<size_t>(q >> qs_shift) * g.W) << qs_shift) + (q & ((1 << qs_shift) - 1));
                k = __ldg(dptr + ((static_cast<size_t>(win0 + w) * WS + j) << qs_shift));
            }
            sts_s32(k_list + e * 4, k);
        }
        if (Cfg::MODE == kModeHigh) {
#pragma unroll 4
            for (int e = tid; e < n_e; e += Cfg::THREADS) {      // a thread revisits its own entries: no barrier in between
                const int v = (e / WS) & 3, w = e / (4 * WS);
                if (v < live_vecs) {
                    const int q = q0 + v, rank = min(max(lds_s32(k_list + e * 4), 0), 63);
                    sts_s32(k_list + e * 4, __ldg(g.cinfo + (static_cast<size_t>(q >> qs_shift) * g.sched.n_win + (win0 + w)) * 64 + rank));
                }
            }
        }
        for (int e = tid; e < n_e; e += Cfg::THREADS)      // an index outside the window reads inside the slot all the same
            sts_s32(k_list + e * 4, min(max(lds_s32(k_list + e * 4), 0), KS - 1));
    }
    __syncthreads();

    float acc[MB][4][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int nb = 0; nb < 4; ++nb)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mb][nb][c] = 0.f;

    bool alive = true;
    for (int it = 0; it < n_win; ++it) {
        const int s = it % STAGES;
        const bool ok = mbar_wait_bounded(bar_full + s * 8, (it / STAGES) & 1, abort_word);
        if (!__syncthreads_and(ok)) { alive = false; break; }
        if (warp < live_vecs) {
            const uint32_t as = ring + s * Cfg::STAGE_BYTES, bs = as + Cfg::A_BYTES + warp * (WS * 128);
            const uint32_t kl = k_list + ((it * 4 + warp) * WS) * 4;
#pragma unroll
            for (int grp = 0; grp < Cfg::GROUPS; ++grp) {
                const int w0 = grp * 8 + t, w1 = w0 + 4;   // kept rows behind fragment columns t and t + 4
                const int k0 = lds_s32(kl + w0 * 4), k1 = lds_s32(kl + w1 * 4);
                uint32_t a[MB][4];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    if (Cfg::A_PLAIN) {                    // rows of 64 bytes: the four k of a fragment column meet in pairs of banks at worst
                        a[mb][0] = lds_u32(as + k0 * 64 + gq * 4);
                        a[mb][1] = lds_u32(as + k0 * 64 + (gq + 8) * 4);
                        a[mb][2] = lds_u32(as + k1 * 64 + gq * 4);
                        a[mb][3] = lds_u32(as + k1 * 64 + (gq + 8) * 4);
                        continue;
                    }
                    // rows mb * 16 + gq and + 8 of the tile: block mb / 2, 32-byte chunks 2 (mb % 2) and + 1
                    const uint32_t blk = as + (mb >> 1) * (KS * 128) + gq * 4, c = (mb & 1) * 2;
                    a[mb][0] = lds_u32(blk + k0 * 128 + ((c ^ (k0 & 3)) << 5));
                    a[mb][1] = lds_u32(blk + k0 * 128 + (((c + 1) ^ (k0 & 3)) << 5));
                    a[mb][2] = lds_u32(blk + k1 * 128 + ((c ^ (k1 & 3)) << 5));
                    a[mb][3] = lds_u32(blk + k1 * 128 + (((c + 1) ^ (k1 & 3)) << 5));
                }
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    const uint32_t b0 = lds_u32(bs + w0 * 128 + ((nb ^ (w0 & 3)) << 5) + gq * 4);
                    const uint32_t b1 = lds_u32(bs + w1 * 128 + ((nb ^ (w1 & 3)) << 5) + gq * 4);
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) mma_tf32_16x8x8(acc[mb][nb], a[mb], b0, b1);
                }
            }
        }
        __syncthreads();                                   // the slot has been read by everyone
        if (tid == 0 && it + STAGES < n_win) fill(it + STAGES);
    }
    grid_launch_dependents();                              // only stores are left
    if (!alive) {
        if (tid == 0) atomicMax(g.status, kDevTimeoutFull);
        return;
    }
    if (warp >= live_vecs) return;

    // accumulator fragment: rows gq and gq + 8 of each 16-row block, columns 2 t and 2 t + 1 of each n8 block
    const int col = warp * 32 + 2 * t;
    if (S > 1) {
        float* slot = g.partial + static_cast<size_t>(blockIdx.x) * (MS * NS);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                float* p = slot + static_cast<size_t>(mb * 16 + gq) * NS + col + nb * 8;
                __stcg(reinterpret_cast<float2*>(p), make_float2(acc[mb][nb][0], acc[mb][nb][1]));
                __stcg(reinterpret_cast<float2*>(p + 8 * NS), make_float2(acc[mb][nb][2], acc[mb][nb][3]));
            }
    } else {
        for (int o = 0; o < outs.n_out; ++o) {
            float* C = output_of(g, outs, o) + outs.col0 + bj + col;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const int r0 = mb * 16 + gq, r1 = r0 + 8;
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    if (r0 < g.M) *reinterpret_cast<float2*>(C + static_cast<size_t>(r0) * outs.ldc + nb * 8) = make_float2(acc[mb][nb][0], acc[mb][nb][1]);
                    if (r1 < g.M) *reinterpret_cast<float2*>(C + static_cast<size_t>(r1) * outs.ldc + nb * 8) = make_float2(acc[mb][nb][2], acc[mb][nb][3]);
                }
            }
        }
    }
}

template <int MS, int WS, int KS, int MODE>
static cudaError_t launch_few_rows(const GemmArgs& a, const GemmOutputs& outs, int ctas, cudaStream_t st)
{
    using Cfg = FewRowsCfg<MS, WS, KS, MODE>;
    auto kernel = nm_gemm_tf32_few_rows_kernel<MS, WS, KS, MODE>;
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
    const int K = a.sched.n_win * KS;
    const int lda = outs.lda ? outs.lda : a.M;
    const int a_blocked = (!Cfg::A_PLAIN && lda % 32 == 0) ? 1 : 0;    // columns past lda read as zeros either way
    e = Cfg::A_PLAIN ? encode_tensor_map_2d(&map_a, a.A, lda, K, 16, KS, 0)
                     : (a_blocked ? encode_tensor_map_blocks32(&map_a, a.A, lda, K, KS, Cfg::ABLK)
                                  : encode_tensor_map_2d(&map_a, a.A, lda, K, 32, KS, 1));
    if (e != cudaSuccess) return e;
    e = encode_tensor_map_blocks32(&map_b, a.B, a.N, a.W, WS - (g_test_short_fill ? 1 : 0), 4);   // (test hook, see kernels.h)
    if (e != cudaSuccess) return e;
    return launch_overlapped(kernel, ctas, Cfg::THREADS, Cfg::SMEM_BYTES, st, a, map_a, map_b, outs, a_blocked);
}

#define NMSPMM_FEW_ROWS_VARIANT(NKEEP, MS, WS, KS, MODE)                                                               \
    { NKEEP, WS, KS, MODE, 128, 32, FewRowsCfg<MS, WS, KS, MODE>::SMEM_BYTES, FewRowsCfg<MS, WS, KS, MODE>::STAGES, 128, \
      &launch_few_rows<MS, WS, KS, MODE>, 2, MS }

extern const SlicedVariant kTf32FewRowsVariants[] = {
    NMSPMM_FEW_ROWS_VARIANT(8, 16, 16, 64, kModeHigh),  NMSPMM_FEW_ROWS_VARIANT(8, 32, 16, 64, kModeHigh),
    NMSPMM_FEW_ROWS_VARIANT(8, 64, 16, 64, kModeHigh),  NMSPMM_FEW_ROWS_VARIANT(4, 16, 8, 64, kModeHigh),
    NMSPMM_FEW_ROWS_VARIANT(4, 32, 8, 64, kModeHigh),   NMSPMM_FEW_ROWS_VARIANT(4, 64, 8, 64, kModeHigh),
    NMSPMM_FEW_ROWS_VARIANT(16, 16, 16, 32, kModeLow),  NMSPMM_FEW_ROWS_VARIANT(16, 32, 16, 32, kModeLow),
    NMSPMM_FEW_ROWS_VARIANT(16, 64, 16, 32, kModeLow),  NMSPMM_FEW_ROWS_VARIANT(8, 16, 8, 32, kModeLow),
    NMSPMM_FEW_ROWS_VARIANT(8, 32, 8, 32, kModeLow),    NMSPMM_FEW_ROWS_VARIANT(8, 64, 8, 32, kModeLow),
};
extern const int kFewRowsVariantCount = sizeof(kTf32FewRowsVariants) / sizeof(kTf32FewRowsVariants[0]);

}  // namespace nmspmm
