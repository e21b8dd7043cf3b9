// FFMA multiply variant for 12 kept rows per 32-k window (kModeLow) staged as pairs of
// windows: 24 rows of B and 64 rows of A per stage, half as many CTA barriers per k.
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low12p[] = { NMSPMM_FFMA_VARIANT(kTile128x128, 12, 128, 128, 64, 24, 64, kModeLow) };
extern const int kFfma_low12p_count = sizeof(kFfma_low12p) / sizeof(kFfma_low12p[0]);
}  // namespace nmspmm
