// Epilogue shared by the TF32 tensor-core kernels: accumulators from Tensor Memory to C (or
// to a K slice's scratch slot), 128 x 32 floats per vector.
#pragma once
#include "common.cuh"
#include "gemm_args.h"
#include "tcgen05.cuh"

namespace nmspmm {

constexpr int kTf32PatchBytes = 32 * 144;   // one warp's 32 x 32 transposition patch, rows 144 bytes apart

// Whole warp.  Stores the vectors v_begin .. v_end - 1 of a 128 x NS tile whose accumulators
// sit at TMEM columns 0 .. NS - 1: rows 32 * quad .. 32 * quad + 31 (quad = warp % 4, the
// TMEM lanes this warp may read).  `patch` is kTf32PatchBytes of shared memory private to
// the warp.  A lane holds one row after tcgen05.ld; the patch turns that into 4 rows x 128
// bytes per store instruction.  The eight shared loads of a vector are issued ahead of its
// eight global stores (as a chain of load -> store pairs the same work took three times as
// long).  The peers' copies (fused all-gather) have a loop of their own so that the common
// single-output case is a plain unrolled run.
template <int NS>
__device__ __forceinline__ void tf32_store_vectors(uint32_t tmem, int quad, int lane, int v_begin, int v_end, uint32_t patch,
                                                   const GemmArgs& g, const GemmOutputs& outs, int bi, int bj, bool sliced,
                                                   int slot)
{
    constexpr int MS = 128;
    const int r_sub = lane >> 3, c4 = (lane & 7) * 4;      // store phase: 4 rows x 8 float4 per instruction
    float* const out0 = sliced ? g.partial + static_cast<size_t>(slot) * MS * NS : nullptr;
#pragma unroll 1
    for (int v = v_begin; v < v_end; ++v) {
        uint32_t acc[32];
        tmem_ld_x32(tmem_addr(tmem, quad * 32, v * 32), acc);
        tmem_wait_ld();
        __syncwarp();                                      // the previous vector's reads of the patch are over
#pragma unroll
        for (int x = 0; x < 8; ++x)
            sts_f4(patch + lane * 144 + x * 16,
                   make_float4(__uint_as_float(acc[4 * x]), __uint_as_float(acc[4 * x + 1]), __uint_as_float(acc[4 * x + 2]),
                               __uint_as_float(acc[4 * x + 3])));
        __syncwarp();
#ifndef NMSPMM_TF32_NOSTORE
        float* const base = sliced ? out0 + static_cast<size_t>(quad * 32 + r_sub) * NS + v * 32 + c4
                                   : g.C + static_cast<size_t>(bi + quad * 32 + r_sub) * outs.ldc + outs.col0 + bj + v * 32 + c4;
        const size_t row_step = sliced ? static_cast<size_t>(NS) : static_cast<size_t>(outs.ldc);
        const int rows_left = sliced ? 32 : g.M - (bi + quad * 32 + r_sub);     // rows 4 * i < rows_left exist
        float4 val[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) val[i] = lds_f4(patch + (4 * i + r_sub) * 144 + c4 * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (4 * i < rows_left) *reinterpret_cast<float4*>(base + static_cast<size_t>(4 * i) * row_step) = val[i];
        if (!sliced && outs.n_out > 1) {
            for (int o = 1; o < outs.n_out; ++o) {         // peers' copies of C when gathering
                float* const pb = outs.C_more[o - 1] + (base - g.C);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (4 * i < rows_left) *reinterpret_cast<float4*>(pb + static_cast<size_t>(4 * i) * row_step) = val[i];
            }
        }
#endif
    }
}

}  // namespace nmspmm
