// FFMA multiply variants for 8 kept rows per 32-k window (kModeHigh): 16 rows of B and
// 64 rows of A per staged window (one merged window).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_high8[] = { NMSPMM_FFMA_TILES(8, 16, 64, kModeHigh) };
extern const int kFfma_high8_count = sizeof(kFfma_high8) / sizeof(kFfma_high8[0]);
}  // namespace nmspmm
