// FFMA multiply variants with 16 compressed rows per window (kModeLow).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low16[] = { NMSPMM_FFMA_TILES(16, kModeLow) };
extern const int kFfma_low16_count = sizeof(kFfma_low16) / sizeof(kFfma_low16[0]);
}  // namespace nmspmm
