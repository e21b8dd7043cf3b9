// TF32 tensor-core path, second form: the A window used dense, B expanded with zeros.
//
// For the ratios that keep many rows (16:32, 12:32) the per-vector contraction
// C[128 x 32] += A_gathered[128 x WS] . B[WS x 32] is cheaper issued as
//
//     C[128 x 256] += A_window[128 x 32] . Bx[32 x 256]
//
// where column n of Bx holds the WS kept values of column n at the k rows its vector's index
// list names and zeros elsewhere: four M128 N256 K8 instructions per 32-k window instead of
// a gather (four instructions of N = QT * WS) plus QT * WS / 8 small products.  The tensor
// core issues 32 / n_keep times the useful work, at the instruction shape it runs fastest.
// Nothing of A passes through registers; what crosses the load/store pipe per window is the
// kept values themselves (WS x 256 floats read from global memory, written once to shared
// memory) and the zeros that wipe a slot's previous use.
//
//   warp 0      TMA producer: per step one tiled copy of the A window, blocks of 32 floats
//               along m with 32-byte chunks swizzled within 128-byte rows (the layout of an
//               MN-major TF32 operand); A has a ring of its own, deeper than Bx's.
//   warp 1      one elected thread issues the four tcgen05.mma of a step (A and Bx from
//               shared memory) and commits to the two barriers that free the A slot and
//               the Bx slot.
//   warps 2-9   one warp per vector of the tile.  Lane j holds the vector's j-th index of the
//               step, every lane 16 bytes of WS / 4 kept rows, both fetched two steps ahead
//               into registers.  A row of a vector's block of Bx is 128 contiguous bytes, so
//               a warp writes four kept rows per store instruction, conflict-free; the rows of
//               the slot's previous use that the new list does not overwrite are zeroed first
//               (a bit mask per slot remembers them).  The stores of a step do not depend on
//               one another: a lone warp running a chain of dependent address computations
//               took 1100 cycles per step where this takes a fraction of the step.  An
//               index list with a repeated or out-of-range entry takes a slower route that
//               adds repeated rows, so that the result is the same sum the other forms
//               compute.  After the last step the same warps read the accumulators and
//               store C.
// Every wait is bounded; a wait that gives up raises the device status word.
#include <cuda.h>

#include "common.cuh"
#include "gemm_args.h"
#include "kernels.h"
#include "tcgen05.cuh"
#include "tf32_epilogue.cuh"

namespace nmspmm {

template <int NKEEP>
struct Tf32ExpandCfg {
    static constexpr int MS = 128, QT = 8, NS = 256, KW = 32, WS = NKEEP;
    static constexpr int A_BYTES = KW * 512;                 // [4 blocks of 32 rows of the tile][KW][32]
    static constexpr int BX_BYTES = QT * KW * 128;           // [QT][KW][32]
    static constexpr int NA = 6, NB = 3;                     // ring depths: A waits for a copy from L2 / HBM, Bx for its builders
    static constexpr int BUILD_WARPS = QT;
    static constexpr int THREADS = (2 + BUILD_WARPS) * 32;
    static constexpr int PF = 2;                             // steps the builders' loads run ahead
    static constexpr int RING_BYTES = NA * A_BYTES + NB * BX_BYTES;
    static constexpr int CTRL_BYTES = 256;
    static constexpr int SMEM_BYTES = RING_BYTES + CTRL_BYTES + 1024;   // + alignment slack
    static constexpr int TMEM_COLS = 256;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of one CTA");
    static_assert(BUILD_WARPS * kTf32PatchBytes <= RING_BYTES, "the epilogue reuses the rings");
    static_assert((2 * NA + 2 * NB + 1) * 8 + 8 <= CTRL_BYTES, "control block");
};

__device__ __forceinline__ float4 ldg_stream_f4(const float* p)
{
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ int ldg_stream_s32(const int* p)
{
    int v;
    asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

template <int NKEEP>
__global__ void __launch_bounds__(Tf32ExpandCfg<NKEEP>::THREADS, 1)
nm_gemm_tf32_expand_kernel(const GemmArgs g, const __grid_constant__ CUtensorMap map_a, const GemmOutputs outs, const int a_blocked)
{
    using Cfg = Tf32ExpandCfg<NKEEP>;
    constexpr int MS = Cfg::MS, NS = Cfg::NS, QT = Cfg::QT, KW = Cfg::KW, WS = Cfg::WS;
    constexpr int NA = Cfg::NA, NB = Cfg::NB, PF = Cfg::PF;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t ring_a = (smem_u32(smem_raw) + 1023u) & ~1023u;        // swizzle atoms want 1024-byte alignment
    const uint32_t ring_b = ring_a + NA * Cfg::A_BYTES;
    const uint32_t bars = ring_a + Cfg::RING_BYTES;
    const uint32_t bar_full_a = bars, bar_empty_a = bar_full_a + NA * 8;
    const uint32_t bar_full_b = bar_empty_a + NA * 8, bar_empty_b = bar_full_b + NB * 8, bar_acc = bar_empty_b + NB * 8;
    const uint32_t tmem_word = bar_acc + 8, abort_word = tmem_word + 4;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs below n_dp take one whole tile each; the others one K slice of a tile of the
    // partial last wave, whose accumulators go to a scratch slot for the reduction kernel.
    const int n_dp = g.sched.n_dp;
    const bool sliced = static_cast<int>(blockIdx.x) >= n_dp;
    const int n_slices = sliced ? g.sched.split_k : 1;
    const int slot = static_cast<int>(blockIdx.x) - n_dp;
    const int tile = sliced ? n_dp + slot / n_slices : static_cast<int>(blockIdx.x);
    int ty, tx;
    tile_coords(tile, g.tiles_x, (g.M + MS - 1) / MS, ty, tx);
    const int bi = ty * MS, bj = tx * NS;
    int win0, n_win;
    slice_range(g.sched.n_win, n_slices, sliced ? slot % n_slices : 0, win0, n_win);
    const int live_vecs = min(QT, (g.N - bj) / 32);

    if (tid == 0) {
        prefetch_tensor_map(&map_a);
        for (int s = 0; s < NA; ++s) {
            mbar_init(bar_full_a + s * 8, 1);                            // the TMA bytes
            mbar_init(bar_empty_a + s * 8, 1);                           // the commit behind the step's instructions
        }
        for (int s = 0; s < NB; ++s) {
            mbar_init(bar_full_b + s * 8, Cfg::BUILD_WARPS);
            mbar_init(bar_empty_b + s * 8, 1);
        }
        mbar_init(bar_acc, 1);
        sts_volatile_s32(abort_word, 0);
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_word, Cfg::TMEM_COLS);
    {
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);                // Bx starts as all zeros
        for (int o = tid * 16; o < NB * Cfg::BX_BYTES; o += Cfg::THREADS * 16) sts_f4(ring_b + o, z);
        fence_proxy_async();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = static_cast<uint32_t>(lds_volatile_s32(tmem_word));
    grid_dependency_wait();                                // everything above overlapped the tail of the kernel ahead

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        for (int it = 0; it < n_win; ++it) {
            const int s = it % NA;
            if (it >= NA) {
                const bool ok = mbar_wait_bounded(bar_empty_a + s * 8, ((it / NA) - 1) & 1, abort_word);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicMax(g.status, kDevTimeoutEmpty);
                    break;
                }
            }
            const uint32_t dst = ring_a + s * Cfg::A_BYTES, full = bar_full_a + s * 8;
            if (elect_one()) {
                mbar_arrive_expect_tx(full, Cfg::A_BYTES);
                if (a_blocked) {
                    tma_load_3d(dst, &map_a, 0, (win0 + it) * KW, bi >> 5, full);
                } else {                                   // rows not a multiple of 32: four boxes of 32 rows, the ragged one zero-filled
                    for (int mb = 0; mb < 4; ++mb) tma_load_2d(dst + mb * (KW * 128), &map_a, bi + mb * 32, (win0 + it) * KW, full);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ instruction issuer
        const uint32_t idesc = umma_idesc_tf32(128, live_vecs * 32, true);
        bool alive = true;
        for (int t = 0; t < n_win; ++t) {
            const int sa = t % NA, sb = t % NB;
            bool ok = mbar_wait_bounded(bar_full_a + sa * 8, (t / NA) & 1, abort_word);
            ok = ok && mbar_wait_bounded(bar_full_b + sb * 8, (t / NB) & 1, abort_word);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t as = ring_a + sa * Cfg::A_BYTES, bs = ring_b + sb * Cfg::BX_BYTES;
#pragma unroll
                for (int ks = 0; ks < KW / 8; ++ks)
                    umma_tf32_ss(tmem_addr(tmem, 0, 0), umma_desc_mn_tf32(as + ks * 1024, KW * 128, 512),
                                 umma_desc_mn_tf32(bs + ks * 1024, KW * 128, 512), idesc, (t | ks) != 0);
                tc_commit(bar_empty_a + sa * 8);
                tc_commit(bar_empty_b + sb * 8);
            }
            __syncwarp();
        }
        if (!alive && lane == 0) atomicMax(g.status, kDevTimeoutMma);
        if (elect_one()) tc_commit(bar_acc);               // every instruction has completed: the accumulators are final
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ builders of Bx
        const int v = warp - 2;                            // the vector this warp expands
        const bool live = v < live_vecs;
        const int q = (bj >> 5) + v, qs_shift = g.qs_shift;
        const int* const dptr = g.D + ((static_cast<size_t>(q >> qs_shift) * g.W) << qs_shift) + (q & ((1 << qs_shift) - 1)) +
                                (static_cast<size_t>(lane < WS ? lane : 0) << qs_shift);
        // A lane works on 16 bytes: columns 4 * (lane % 8) .. + 3 of the kept rows lane / 8 + 4 i.
        // One warp instruction then covers four rows of 128 bytes, each quarter of the warp
        // one row, and a row of the vector's block is 128 contiguous bytes (eight 16-byte
        // pieces, pairs of them swizzled with the row number): no bank conflicts either way.
        constexpr int RPL = WS / 4;                        // kept rows per lane
        static_assert(WS % 4 == 0, "four kept rows per warp instruction");
        const int quarter = lane >> 3, piece = lane & 7;
        const float* const bptr = g.B + bj + v * 32 + piece * 4;
        auto row_addr = [&](uint32_t block, int k) -> uint32_t {          // this lane's 16 bytes of row k of the vector's block
            return block + k * 128 + (((static_cast<uint32_t>(piece >> 1) ^ (k & 3)) << 5) | ((piece & 1) << 4));
        };
        int idx_r[PF + 1];
        float4 val_r[PF + 1][RPL];
        uint32_t hist[NB];                                 // rows set in the slots, oldest last
#pragma unroll
        for (int i = 0; i < NB; ++i) hist[i] = 0;
        auto fetch = [&](int it, int& idx, float4 (&val)[RPL]) {
            const size_t row0 = static_cast<size_t>(win0 + it) * WS;
            idx = -1;
            if (live && it < n_win) {
                if (lane < WS) idx = ldg_stream_s32(dptr + (row0 << qs_shift));
#pragma unroll
                for (int i = 0; i < RPL; ++i) val[i] = ldg_stream_f4(bptr + (row0 + quarter + 4 * i) * g.N);
            }
        };
#pragma unroll
        for (int p = 0; p < PF; ++p) fetch(p, idx_r[p], val_r[p]);
        bool alive = true;
        // The loop is unrolled over the PF + 1 register sets so that a set is named statically:
        // a value loaded for step it + PF is first touched in step it + PF.
        for (int it0 = 0; it0 < n_win && alive; it0 += PF + 1) {
#pragma unroll
            for (int ph = 0; ph < PF + 1; ++ph) {
                const int it = it0 + ph;
                if (it >= n_win || !alive) continue;
                fetch(it + PF, idx_r[(ph + PF) % (PF + 1)], val_r[(ph + PF) % (PF + 1)]);
                const int sb = it % NB;
                if (it >= NB) {
                    const bool ok = mbar_wait_bounded(bar_empty_b + sb * 8, ((it / NB) - 1) & 1, abort_word);
                    if (!__all_sync(0xffffffffu, ok)) { alive = false; continue; }
                }
                if (live) {
                    const uint32_t block = ring_b + sb * Cfg::BX_BYTES + v * (KW * 128);
                    const int idx = idx_r[ph];
                    const float4(&val)[RPL] = val_r[ph];
                    const bool valid = lane >= WS || static_cast<unsigned>(idx) < static_cast<unsigned>(KW);
                    const uint32_t rows = __reduce_or_sync(0xffffffffu, (lane < WS && valid) ? (1u << idx) : 0u);
                    const bool plain = __all_sync(0xffffffffu, valid) && __popc(rows) == WS;
                    int k[RPL];                            // where this lane's kept rows go
#pragma unroll
                    for (int i = 0; i < RPL; ++i) k[i] = __shfl_sync(0xffffffffu, idx, quarter + 4 * i);
                    // rows of the slot's previous use that the new list does not overwrite: every
                    // quarter of the warp looks at its own row of each group of four
                    const uint32_t wipe = (plain ? (hist[NB - 1] & ~rows) : hist[NB - 1]) >> quarter;
                    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int gi = 0; gi < KW / 4; ++gi)
                        if ((wipe >> (4 * gi)) & 1u) sts_f4(row_addr(block, 4 * gi + quarter), z);
                    if (plain) {
#pragma unroll
                        for (int i = 0; i < RPL; ++i) sts_f4(row_addr(block, k[i]), val[i]);
                    } else {
                        // repeated rows add up, rows outside the window are dropped: one kept row at a
                        // time, so that two quarters never update the same row in one instruction
#pragma unroll
                        for (int i = 0; i < RPL; ++i) {
#pragma unroll
                            for (int qq = 0; qq < 4; ++qq) {
                                if (quarter == qq && static_cast<unsigned>(k[i]) < static_cast<unsigned>(KW)) {
                                    const uint32_t a = row_addr(block, k[i]);
                                    const float4 o = lds_f4(a);
                                    sts_f4(a, make_float4(o.x + val[i].x, o.y + val[i].y, o.z + val[i].z, o.w + val[i].w));
                                }
                                __syncwarp();
                            }
                        }
                    }
#pragma unroll
                    for (int i = NB - 1; i > 0; --i) hist[i] = hist[i - 1];
                    hist[0] = rows;
                }
                fence_proxy_async();                       // the tensor core reads Bx through the asynchronous proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full_b + sb * 8);
            }
        }
        // ------------------------------------------------------------------ epilogue
        bool ok = alive && mbar_wait_bounded(bar_acc, 0, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        grid_launch_dependents();                          // only stores are left
        if (ok) {
            tc_fence_after_sync();
            // every instruction has completed, so every copy has landed and been read: the
            // rings are free and serve as the transposition patches.  Two warps share a TMEM
            // lane quadrant (warp % 4); each takes half of the tile's vectors.
            const int half = v >> 2;
            tf32_store_vectors<NS>(tmem, warp & 3, lane, min(half * (QT / 2), live_vecs), min((half + 1) * (QT / 2), live_vecs),
                                   ring_a + v * kTf32PatchBytes, g, outs, bi, bj, sliced, slot);
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

template <int NKEEP>
static cudaError_t launch_tf32_expand(const GemmArgs& a, const GemmOutputs& outs, int tiles, cudaStream_t st)
{
    using Cfg = Tf32ExpandCfg<NKEEP>;
    auto kernel = nm_gemm_tf32_expand_kernel<NKEEP>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    CUtensorMap map_a;
    const int K = a.sched.n_win * Cfg::KW;
    const int lda = outs.lda ? outs.lda : a.M;             // a row-major caller's transposed copy is padded to 4 columns
    const int a_blocked = (lda % 32 == 0) ? 1 : 0;
    const int box_rows = Cfg::KW - (g_test_short_fill ? 1 : 0);          // (test hook, see kernels.h)
    e = a_blocked ? encode_tensor_map_blocks32(&map_a, a.A, lda, K, box_rows, 4)
                  : encode_tensor_map_2d(&map_a, a.A, lda, K, 32, box_rows, 1);
    if (e != cudaSuccess) return e;
    return launch_overlapped(kernel, tiles, Cfg::THREADS, Cfg::SMEM_BYTES, st, a, map_a, outs, a_blocked);
}

#define NMSPMM_TF32_EXPAND_VARIANT(NKEEP)                                                                              \
    { NKEEP, Tf32ExpandCfg<NKEEP>::WS, 32, kModeLow, 256, 32, Tf32ExpandCfg<NKEEP>::SMEM_BYTES, Tf32ExpandCfg<NKEEP>::NA,   \
      Tf32ExpandCfg<NKEEP>::THREADS, &launch_tf32_expand<NKEEP>, 1 }

extern const SlicedVariant kTf32ExpandVariants[] = {
    NMSPMM_TF32_EXPAND_VARIANT(16), NMSPMM_TF32_EXPAND_VARIANT(12), NMSPMM_TF32_EXPAND_VARIANT(8),
};
extern const int kTf32ExpandVariantCount = sizeof(kTf32ExpandVariants) / sizeof(kTf32ExpandVariants[0]);


}  // namespace nmspmm
