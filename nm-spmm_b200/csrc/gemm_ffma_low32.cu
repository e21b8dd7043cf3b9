// FFMA multiply variants for 32 kept rows per 32-k window (kModeLow): 32 rows of B and
// 32 rows of A per staged window.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low32[] = { NMSPMM_FFMA_TILES(32, 32, 32, kModeLow) };
extern const int kFfma_low32_count = sizeof(kFfma_low32) / sizeof(kFfma_low32[0]);
}  // namespace nmspmm
