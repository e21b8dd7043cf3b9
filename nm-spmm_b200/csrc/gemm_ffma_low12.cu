// FFMA multiply variants for 12 kept rows per 32-k window (kModeLow): 12 rows of B and
// 32 rows of A per staged window.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low12[] = { NMSPMM_FFMA_TILES(12, 12, 32, kModeLow) };
extern const int kFfma_low12_count = sizeof(kFfma_low12) / sizeof(kFfma_low12[0]);
}  // namespace nmspmm
