// Internal host-side declarations shared by the library's translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "gemm_args.h"

namespace nmspmm {

cudaError_t launch_trans_index(int* DT, int W, int Q, int pruning_N, int pruning_M, cudaStream_t st);
cudaError_t launch_retile(const int* DT, int* D, int W, int Q, int Qs, cudaStream_t st);
cudaError_t launch_preprocess_high(const int* DT, int* D, int* cinfo, int pm, int pn, int W, int Q, int Qs,
                                   int fuse, int tail_ints, cudaStream_t st);

// in [M][K] row-major -> out [K][ld] (ld >= M, the extra columns zero).
cudaError_t launch_transpose_rows(const float* in, float* out, int M, int K, int ld, cudaStream_t st);

// 16-bit storage (convert16.cu): the same transposition from half / bfloat16 rows, n floats
// rounded to 16 bits, n 16-bit values widened (n % 4 == 0).
enum { kDtypeF32 = 0, kDtypeF16 = 1, kDtypeBF16 = 2 };
cudaError_t launch_transpose_rows_16(int dtype, const void* in, float* out, int M, int K, int ld, cudaStream_t st);
cudaError_t launch_narrow(int dtype, const float* in, void* out, size_t n, cudaStream_t st);
cudaError_t launch_widen(int dtype, const void* in, float* out, size_t n, cudaStream_t st);

// One compiled FFMA kernel variant.
struct FfmaVariant {
    int tile_id;        // nmspmm_tile
    int ms, ns;         // CTA tile
    int n_keep;         // kept rows per 32-k window this variant is compiled for
    int ws;             // compressed rows of B per staged window
    int ks;             // rows of A per staged window (32, or 64: a merged HIGH window)
    int mode;           // kModeLow / kModeHigh
    int threads, smem_bytes, stages, min_blocks;
    cudaError_t (*launch)(const GemmArgs&, const GemmOutputs&, int grid, cudaStream_t st);         // private M x N matrix args.C
    cudaError_t (*launch_multi)(const GemmArgs&, const GemmOutputs&, int grid, cudaStream_t st);   // every output at (ldc, col0)
};
// Returns nullptr when the combination was not compiled.
const FfmaVariant* find_ffma_variant(int tile_id, int n_keep, int mode);

// Row-major 2-D float tensor [rows][cols] (cols innermost) with a box_cols x box_rows box;
// swizzle128 = 0: rows land unswizzled, 1: 32-byte chunks swizzled within 128-byte rows
// (CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B; box_cols * 4 must be 128).
// Elements outside the tensor are delivered as zeros.
cudaError_t encode_tensor_map_2d(CUtensorMap* map, const float* base, int cols, int rows, int box_cols, int box_rows,
                                 int swizzle128 = 0);

// Row-major [rows][cols] float tensor as blocks of 32 columns (cols % 32 == 0): a box of
// box_blocks blocks x box_rows rows lands block after block, each [box_rows][32] swizzled like
// encode_tensor_map_2d's swizzle128 form.
cudaError_t encode_tensor_map_blocks32(CUtensorMap* map, const float* base, int cols, int rows, int box_rows, int box_blocks);

// One compiled variant of the kernels that cut K into whole slices per tile and leave the
// slices in scratch slots for nm_reduce_slices_kernel: the TF32 tensor-core kernels (tile
// 128 x ns) and the few-rows kernels (tile ms x 128).
struct SlicedVariant {
    int n_keep;         // kept rows per 32-k window
    int ws, ks;         // rows of B / of A per step
    int mode;
    int ns;             // tile columns: 256 (one CTA per SM) or 128 (two)
    int vec_len;        // columns that share an index list: 32, or 64 (adjacent equal lists)
    int smem_bytes, stages, threads;
    cudaError_t (*launch)(const GemmArgs&, const GemmOutputs&, int tiles, cudaStream_t st);
    int form;           // 0: A gathered by the tensor core, 1: B expanded with zeros, 2: few rows on warp-level MMA
    int ms;             // tile rows when not 128 (form 2: 16, 32 or 64), else 0
};
extern const SlicedVariant kTf32GatherVariants[];
extern const int kTf32GatherVariantCount;
extern const SlicedVariant kTf32FewRowsVariants[];  // few rows of A on warp-level MMA (gemm_tf32_few_rows.cu)
extern const int kFewRowsVariantCount;
constexpr int kFewRowsMaxWindows = 24;              // k windows one CTA of that form takes (its resolved index list is in shared memory)
extern const SlicedVariant kTf32ExpandVariants[];   // the form that expands B with zeros (gemm_tf32_expand.cu)
extern const int kTf32ExpandVariantCount;

// Adds the pieces the multiply left in scratch (args.counters == nullptr) for the tiles
// first_tile .. first_tile + n_tiles - 1 of the given CTA tile and writes C.
cudaError_t launch_reduce_pieces(int tile_id, const GemmArgs& args, const GemmOutputs& outs, int first_tile, int n_tiles,
                                 cudaStream_t st);

// Adds the K slices the tensor-core multiply (tile 128 x ns) left in scratch for the tiles
// first_tile .. first_tile + n_tiles - 1 (args.sched.split_k slices each) and writes C.
cudaError_t launch_reduce_slices(int ns, const GemmArgs& args, const GemmOutputs& outs, int first_tile, int n_tiles,
                                 cudaStream_t st, int ms = 128);

// Launch with programmatic stream serialisation: the grid may be set up, and its CTAs may run
// up to their griddepcontrol.wait, while the kernel ahead of it on the stream is still
// finishing.  Every kernel launched this way executes griddepcontrol.wait before its first
// access to global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned blocks, unsigned threads, size_t smem_bytes,
                                     cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Test hook (nmspmm_test_short_fill): non-zero makes the multiply launchers encode B's tensor
// map (A's in gemm_tf32_expand.cu, which loads B without TMA) with a box one row short.  The kernels are unchanged; their stages then never fill.
extern int g_test_short_fill;

// packed = 0: scalar FFMA loop; 1: two-lane packed FFMA2 loop.
cudaError_t measure_ffma_peak(double* tflops, int packed, cudaStream_t st);

}  // namespace nmspmm
