// Tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

#include "kernels.h"

namespace nmspmm {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

cudaError_t encode_tensor_map_2d(CUtensorMap* map, const float* base, int cols, int rows, int box_cols, int box_rows,
                                 int swizzle128)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = { static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows) };
    const cuuint64_t strides[1] = { static_cast<cuuint64_t>(cols) * sizeof(float) };
    const cuuint32_t box[2] = { static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows) };
    const cuuint32_t elem[2] = { 1, 1 };
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// The same row-major [rows][cols] tensor seen as blocks of 32 columns: dimensions
// {32 columns, rows, cols / 32 blocks}, box {32, box_rows, box_blocks}.  A box lands in
// shared memory block after block, each block [box_rows][32] with its 32-byte chunks
// swizzled within the 128-byte rows: the layout of an MN-major TF32 tensor-core operand
// that is box_blocks * 32 values wide.  cols must be a multiple of 32 (a partial last block
// would run on into the next row instead of reading as zeros).
cudaError_t encode_tensor_map_blocks32(CUtensorMap* map, const float* base, int cols, int rows, int box_rows, int box_blocks)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cudaErrorNotSupported;
    if (cols % 32 != 0) return cudaErrorInvalidValue;
    const cuuint64_t dims[3] = { 32, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(cols / 32) };
    const cuuint64_t strides[2] = { static_cast<cuuint64_t>(cols) * sizeof(float), 32 * sizeof(float) };
    const cuuint32_t box[3] = { 32, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_blocks) };
    const cuuint32_t elem[3] = { 1, 1, 1 };
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace nmspmm
