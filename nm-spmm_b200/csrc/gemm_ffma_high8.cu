// FFMA multiply variants with 8 compressed rows per window (kModeHigh).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_high8[] = { NMSPMM_FFMA_TILES(8, kModeHigh) };
extern const int kFfma_high8_count = sizeof(kFfma_high8) / sizeof(kFfma_high8[0]);
}  // namespace nmspmm
