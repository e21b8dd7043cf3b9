// FFMA multiply variants with 8 compressed rows per window (kModeLow).
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low8[] = { NMSPMM_FFMA_TILES(8, kModeLow) };
extern const int kFfma_low8_count = sizeof(kFfma_low8) / sizeof(kFfma_low8[0]);
}  // namespace nmspmm
