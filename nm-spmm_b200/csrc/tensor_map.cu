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

// Encoding a tensor map costs about a microsecond of host time, and a caller in a loop asks
// for the same few over and over (same operands, same tiles).  The last few encodings of each
// host thread are kept, keyed by everything that goes into them.
struct MapKey {
    const void* base;
    int cols, rows, box_a, box_b, kind;       // kind: 0 plain 2-D, 1 swizzled 2-D, 2 blocks of 32 columns
    bool operator==(const MapKey& o) const
    {
        return base == o.base && cols == o.cols && rows == o.rows && box_a == o.box_a && box_b == o.box_b && kind == o.kind;
    }
};
struct MapCache {
    static constexpr int kEntries = 8;
    MapKey key[kEntries] = {};
    CUtensorMap map[kEntries];
    bool used[kEntries] = {};
    int next = 0;
    bool find(const MapKey& k, CUtensorMap* out) const
    {
        for (int i = 0; i < kEntries; ++i)
            if (used[i] && key[i] == k) {
                *out = map[i];
                return true;
            }
        return false;
    }
    void put(const MapKey& k, const CUtensorMap& m)
    {
        key[next] = k;
        map[next] = m;
        used[next] = true;
        next = (next + 1) % kEntries;
    }
};
static thread_local MapCache tl_maps;

cudaError_t encode_tensor_map_2d(CUtensorMap* map, const float* base, int cols, int rows, int box_cols, int box_rows,
                                 int swizzle128)
{
    const MapKey mk { base, cols, rows, box_cols, box_rows, swizzle128 ? 1 : 0 };
    if (tl_maps.find(mk, map)) return cudaSuccess;
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
    if (r == CUDA_SUCCESS) tl_maps.put(mk, *map);
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
    const MapKey mk { base, cols, rows, box_rows, box_blocks, 2 };
    if (tl_maps.find(mk, map)) return cudaSuccess;
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
    if (r == CUDA_SUCCESS) tl_maps.put(mk, *map);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace nmspmm
