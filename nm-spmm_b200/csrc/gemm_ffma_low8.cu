// FFMA multiply variants for 8 kept rows per 32-k window (kModeLow): 8 rows of B and
// 32 rows of A per staged window.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low8[] = { NMSPMM_FFMA_TILES(8, 8, 32, kModeLow) };
extern const int kFfma_low8_count = sizeof(kFfma_low8) / sizeof(kFfma_low8[0]);
}  // namespace nmspmm
