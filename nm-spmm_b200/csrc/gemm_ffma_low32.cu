// FFMA multiply variants with 32 compressed rows per window (kModeLow).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low32[] = { NMSPMM_FFMA_TILES(32, kModeLow) };
extern const int kFfma_low32_count = sizeof(kFfma_low32) / sizeof(kFfma_low32[0]);
}  // namespace nmspmm
