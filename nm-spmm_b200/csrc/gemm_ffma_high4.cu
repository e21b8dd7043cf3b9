// FFMA multiply variants for 4 kept rows per 32-k window (kModeHigh): 8 rows of B and
// 64 rows of A per staged window.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_high4[] = { NMSPMM_FFMA_TILES(4, 8, 64, kModeHigh) };
extern const int kFfma_high4_count = sizeof(kFfma_high4) / sizeof(kFfma_high4[0]);
}  // namespace nmspmm
