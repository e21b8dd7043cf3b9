// FFMA multiply variants with 16 compressed rows per window (kModeHigh).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_high16[] = { NMSPMM_FFMA_TILES(16, kModeHigh) };
extern const int kFfma_high16_count = sizeof(kFfma_high16) / sizeof(kFfma_high16[0]);
}  // namespace nmspmm
