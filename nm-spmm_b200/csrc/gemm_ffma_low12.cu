// FFMA multiply variants with 12 compressed rows per window (kModeLow).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low12[] = { NMSPMM_FFMA_TILES(12, kModeLow) };
extern const int kFfma_low12_count = sizeof(kFfma_low12) / sizeof(kFfma_low12[0]);
}  // namespace nmspmm
