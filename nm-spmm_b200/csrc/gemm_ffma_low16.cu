// FFMA multiply variants for 16 kept rows per 32-k window (kModeLow): 16 rows of B and
// 32 rows of A per staged window.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low16[] = { NMSPMM_FFMA_TILES(16, 16, 32, kModeLow) };
extern const int kFfma_low16_count = sizeof(kFfma_low16) / sizeof(kFfma_low16[0]);
}  // namespace nmspmm
