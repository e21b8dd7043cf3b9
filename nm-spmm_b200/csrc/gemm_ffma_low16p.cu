// FFMA multiply variant for 16 kept rows per 32-k window (kModeLow) staged as pairs of
// windows: 32 rows of B and 64 rows of A per stage, half as many CTA barriers per k.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low16p[] = { NMSPMM_FFMA_VARIANT(kTile128x128, 16, 128, 128, 64, 32, 64, kModeLow) };
extern const int kFfma_low16p_count = sizeof(kFfma_low16p) / sizeof(kFfma_low16p[0]);
}  // namespace nmspmm
